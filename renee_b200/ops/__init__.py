"""Fused ops of the package: one entry point per op, writing into caller-provided buffers.

CUDA tensors are served by the hand-written sm_100a kernels of ``renee_b200/ops/csrc`` (loaded
from the in-tree shared library through :mod:`renee_b200.ops.cuda`); CPU tensors are served by the
PyTorch oracles of :mod:`renee_b200.ops.reference`.  A CUDA tensor with a missing or stale kernel
library is an error, never a silent fallback.

All functions take an ``rng`` handle (:class:`StepRNG`) rather than a raw seed: the CPU path reads
``rng.seed`` (a Python int), the kernels read the seed from device memory (``rng.dev``), which keeps
a captured CUDA graph valid when the seed changes every step.
"""
from __future__ import annotations

import torch

from . import reference as ref
from ..utils import guard
from .rng import DropoutRNG, keep_mask  # noqa: F401


class StepRNG:
    """Per-step dropout seed: ``seed`` for the CPU oracles, ``dev`` (int32 tensor ``[1]`` on the
    device holding the same value) for the kernels."""

    def __init__(self, seed: int = 0, dev: torch.Tensor | None = None):
        self.seed = int(seed)
        self.dev = dev

    def set(self, seed: int) -> None:
        self.seed = int(seed) & 0xFFFFFFFF


def _cuda():
    from . import cuda as cu
    return cu


def _is_cuda(t: torch.Tensor) -> bool:
    return t.is_cuda


# ----------------------------------------------------------------------------- encoder ops
def embed_ln_fwd(ids, word, pos, gamma, beta, eps, S, p, rng, stream, out, mean, rstd):
    if _is_cuda(out):
        return _cuda().embed_ln_fwd(ids, word, pos, gamma, beta, eps, S, p, rng, stream, out, mean, rstd)
    y, m, r = ref.embed_ln_fwd(ids, word, pos, gamma, beta, eps, S, p, rng.seed, stream, out.dtype)
    out.copy_(y); mean.copy_(m); rstd.copy_(r)


def embed_ln_bwd(dy, ids, word, pos, gamma, mean, rstd, S, p, rng, stream, pad_id, dword, dpos, dgamma, dbeta):
    if _is_cuda(dy):
        return _cuda().embed_ln_bwd(dy, ids, word, pos, gamma, mean, rstd, S, p, rng, stream, pad_id,
                                    dword, dpos, dgamma, dbeta)
    ref.embed_ln_bwd(dy, ids, word, pos, gamma, mean, rstd, S, p, rng.seed, stream, pad_id, dword, dpos, dgamma, dbeta)


def attention_workspace(b, S, nh, device, dtype, ds=None):
    """Buffers the attention forward leaves for its backward: the softmax probabilities.  On CUDA, 16-bit
    sequences longer than 128 tokens also need a same-shaped scratch for the softmax gradient (``ds``; pass one
    tensor to share it between layers, it only lives within one backward call)."""
    ws = {"probs": guard.empty(b, nh, S, S, dtype=dtype, device=device, name="attention.probs")}
    if S > 128 and torch.device(device).type == "cuda" and dtype != torch.float32:
        ws["ds"] = ds if ds is not None else guard.empty(b, nh, S, S, dtype=dtype, device=device, name="attention.ds")
    return ws


def attention_fwd(qkv, bqkv, mask, nh, p, rng, stream, ctx_out, ws):
    b = mask.shape[0]
    if _is_cuda(qkv):
        return _cuda().attention_fwd(qkv, bqkv, mask, nh, p, rng, stream, ctx_out, ws)
    ctx, probs = ref.attention_fwd(qkv, bqkv, mask, nh, p, rng.seed, stream)
    ctx_out.copy_(ctx)
    ws["probs"][:b].copy_(probs)


def attention_bwd(dctx, qkv, bqkv, mask, nh, p, rng, stream, ws, dqkv_out, dbqkv_out):
    b = mask.shape[0]
    if _is_cuda(qkv):
        return _cuda().attention_bwd(dctx, qkv, bqkv, mask, nh, p, rng, stream, ws, dqkv_out, dbqkv_out)
    d = ref.attention_bwd(dctx, qkv, bqkv, mask, ws["probs"][:b], nh, p, rng.seed, stream)
    dqkv_out.copy_(d)
    ref.colsum(d, dbqkv_out)


def bias_dropout_add_ln_fwd(x, bias, resid, gamma, beta, eps, p, rng, stream, y_out, pre_out, mean, rstd):
    if _is_cuda(x):
        return _cuda().bias_dropout_add_ln_fwd(x, bias, resid, gamma, beta, eps, p, rng, stream,
                                               y_out, pre_out, mean, rstd)
    y, pre, m, r = ref.bias_dropout_add_ln_fwd(x, bias, resid, gamma, beta, eps, p, rng.seed, stream)
    y_out.copy_(y); pre_out.copy_(pre); mean.copy_(m); rstd.copy_(r)


def bias_dropout_add_ln_bwd(dy, pre, gamma, mean, rstd, p, rng, stream, dgamma, dbeta, dbias,
                            dpre_out, dbranch_out):
    """Returns ``(d_pre, d_branch)``; with ``p == 0`` both are the same tensor (``dpre_out``)."""
    if _is_cuda(dy):
        return _cuda().bias_dropout_add_ln_bwd(dy, pre, gamma, mean, rstd, p, rng, stream,
                                               dgamma, dbeta, dbias, dpre_out, dbranch_out)
    d_pre, d_branch = ref.bias_dropout_add_ln_bwd(dy, pre, gamma, mean, rstd, p, rng.seed, stream,
                                                  dgamma, dbeta, dbias)
    dpre_out.copy_(d_pre)
    if p > 0:
        dbranch_out.copy_(d_branch)
        return dpre_out, dbranch_out
    return dpre_out, dpre_out


def bias_gelu_fwd(x, bias, out):
    if _is_cuda(x):
        return _cuda().bias_gelu_fwd(x, bias, out)
    out.copy_(ref.bias_gelu_fwd(x, bias))


def bias_gelu_bwd(da, x, bias, dbias, dx_out):
    if _is_cuda(x):
        return _cuda().bias_gelu_bwd(da, x, bias, dbias, dx_out)
    dx_out.copy_(ref.bias_gelu_bwd(da, x, bias, dbias))


def pool_fwd(h, mask, mode, out):
    if _is_cuda(h):
        return _cuda().pool_fwd(h, mask, mode, out)
    out.copy_(ref.pool_fwd(h, mask, mode))


def pool_bwd(de, mask, mode, S, dh_out):
    if _is_cuda(de):
        return _cuda().pool_bwd(de, mask, mode, S, dh_out)
    dh_out.copy_(ref.pool_bwd(de, mask, mode, S, dh_out.dtype))


def dropout_cast_fwd(e, p, rng, stream, out):
    if _is_cuda(e):
        return _cuda().dropout_cast_fwd(e, p, rng, stream, out)
    out.copy_(ref.dropout_cast_fwd(e, p, rng.seed, stream, out.dtype))


def dropout_bwd(dx, p, rng, stream, out):
    if _is_cuda(dx):
        return _cuda().dropout_bwd(dx, p, rng, stream, out)
    out.copy_(ref.dropout_bwd(dx, p, rng.seed, stream))


# ----------------------------------------------------------------------------- optimizer
def adamw_step(p32, m, v, g, p16, hp, beta1, beta2, eps, wd, n_decay, grad_mult=1.0):
    """``hp`` is the device-resident hyper-parameter block (see :mod:`renee_b200.optim.hparams`):
    learning rate, Adam step count, inverse loss scale and the found-inf flag are read from it."""
    if _is_cuda(p32):
        return _cuda().adamw_step(p32, m, v, g, p16, hp, beta1, beta2, eps, wd, n_decay, grad_mult)
    from ..optim.hparams import HP
    h = hp.buf
    ref.adamw_step(p32, m, v, g, None if p16 is p32 else p16, float(h[HP.LR_ENC]), beta1, beta2, eps, wd, n_decay,
                   float(h[HP.ADAM_STEP]) + 1.0, float(h[HP.INV_SCALE]) * grad_mult, float(h[HP.FOUND_INF]))
