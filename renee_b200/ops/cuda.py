"""ctypes bindings of the in-tree sm_100a kernel library (``_kernels.so``).

Loading fails loudly: a CUDA tensor reaching :mod:`renee_b200.ops` without a current library is an
error, not a fallback.  Every wrapper launches on PyTorch's current stream and performs no
allocation and no host synchronisation, so whole training steps can be captured in a CUDA graph.
``launch_count()`` reports how many kernels of this library were launched (``bench.py`` uses it).
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import build as _build

_LIB = None
_LAUNCHES = 0
_c = ctypes
_VP, _I, _F, _LL, _U = _c.c_void_p, _c.c_int, _c.c_float, _c.c_longlong, _c.c_uint

DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


class KernelError(RuntimeError):
    pass


def lib():
    global _LIB
    if _LIB is None:
        _load()
    return _LIB


LN_BWD_WARPS = 4     # warps per CTA of the LayerNorm backward kernel (4, 8 or 16; RENEE_B200_LN_BWD_WARPS overrides).  Measured:
                     # 8192 x 768 alone 34.9 / 29.2 / 30.6 us with 4 / 8 / 16, but the training step does not gain (3.75 /
                     # 3.74 / 3.73 ms at 8192 tokens) and loses 5 % at 4096 tokens per GPU (2.43 / 2.56 / 2.57 ms)


def _load():
    global _LIB
    if not _build.is_current():
        if os.environ.get("RENEE_B200_NO_BUILD") == "1" or not _has_nvcc():
            if not os.path.exists(_build.LIB):
                raise KernelError(f"{_build.LIB} is missing and cannot be built here; run "
                                  "`python -m renee_b200.ops.build`")
        else:
            _build.build()
    _LIB = ctypes.CDLL(_build.LIB)
    if os.environ.get("RENEE_B200_PDL", "1") == "0":
        _LIB.rb_enc_gemm_set_pdl(_I(0))
    _LIB.rb_set_ln_bwd_warps(_I(int(os.environ.get("RENEE_B200_LN_BWD_WARPS", LN_BWD_WARPS))))
    if os.environ.get("RENEE_B200_GEMM_MAX_UNITS"):
        _LIB.rb_enc_gemm_set_max_units(_I(int(os.environ["RENEE_B200_GEMM_MAX_UNITS"])))


def _has_nvcc() -> bool:
    try:
        _build.nvcc_path()
        return True
    except RuntimeError:
        return False


def launch_count() -> int:
    return _LAUNCHES


def _stream():
    return _VP(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return _VP(0) if t is None else _VP(t.data_ptr())


def _call(name, *args, launches=1):
    global _LAUNCHES
    rc = getattr(lib(), name)(*args)
    if rc != 0:
        raise KernelError(f"{name} failed with code {rc}")
    _LAUNCHES += launches


# ----------------------------------------------------------------------------- workspaces
class _Workspace:
    """Small per-device scratch: fp32 column accumulators (zero between calls by contract of the
    kernels), block counters, and the status words the bounded waits write."""

    def __init__(self, device):
        self.colacc = torch.zeros(8 * 3 * 8192, dtype=torch.float32, device=device)   # 8 replicas x 3 vectors x max width
        self.counters = torch.zeros(16, dtype=torch.int32, device=device)
        self.status = torch.zeros(8, dtype=torch.int32, device=device)


_WS: dict = {}


def workspace(device) -> _Workspace:
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _WS:
        _WS[key] = _Workspace(torch.device("cuda", key))
    return _WS[key]


def check_status(device=None) -> None:
    """Raise if any bounded device-side wait has timed out since the last check (synchronises)."""
    ws = workspace(device if device is not None else torch.cuda.current_device())
    st = ws.status.cpu().tolist()
    if st[0] != 0:
        ws.status.zero_()
        raise KernelError(f"device-side wait timed out: code={st[0]} block={st[1]} site={st[2]} detail={st[3]}")


# ----------------------------------------------------------------------------- deferred column sums
class DeferredColumns:
    """Per-engine plan for the column reductions of a backward pass (LayerNorm gamma/beta and all bias
    gradients).  While a plan is active, the kernels only accumulate into their own fp32 replica block and
    skip their last-block finalize; ``finalize()`` converts everything with one launch.  Slots are keyed by
    the output addresses (views of the flat gradient buffer, stable across steps), so after the first
    step no allocation happens and the launch sequence can be captured in a CUDA graph."""

    REPLICAS = 8

    def __init__(self, device, dtype):
        self.device, self.dtype = device, dtype
        self.slots: dict = {}
        self.rows: list = []
        self.table = None
        self.max_len = 0

    def slot(self, outs, width: int) -> torch.Tensor:
        key = tuple(0 if o is None else o.data_ptr() for o in outs) + (width,)
        acc = self.slots.get(key)
        if acc is None:
            n_vec = len(outs)
            acc = torch.zeros(self.REPLICAS * n_vec * width, dtype=torch.float32, device=self.device)
            self.slots[key] = acc
            for v, o in enumerate(outs):
                if o is not None:
                    self.rows.append((acc.data_ptr(), o.data_ptr(), n_vec * width, v * width, width))
            self.max_len = max(self.max_len, width)
            self.table = None
        return acc

    def finalize(self) -> None:
        if not self.rows:
            return
        if self.table is None:
            import numpy as np
            t = np.zeros((len(self.rows), 4), dtype=np.int64)
            for i, (a, o, tot, voff, n) in enumerate(self.rows):
                t[i] = (a, o, tot | (voff << 32), n)      # {acc*, out*, int tot, int v_off, int len, int pad}
            self.table = torch.from_numpy(t).to(self.device)
        _call("rb_finalize_columns", _I(DT[self.dtype]), _p(self.table), _I(len(self.rows)), _I(self.max_len), _stream())


_DEFER: DeferredColumns | None = None


class deferred_columns:
    def __init__(self, plan: DeferredColumns | None):
        self.plan = plan

    def __enter__(self):
        global _DEFER
        self.prev, _DEFER = _DEFER, self.plan
        return self.plan

    def __exit__(self, *exc):
        global _DEFER
        _DEFER = self.prev
        return False


def _acc_for(outs, width, default_counter):
    """(accumulator, counter) for a column-reducing kernel: the active plan's slot (no counter → no
    in-kernel finalize) or the shared workspace with the kernel's own counter."""
    if _DEFER is not None:
        return _DEFER.slot(outs, width), None
    ws = workspace(outs[0].device if outs[0] is not None else torch.cuda.current_device())
    if DeferredColumns.REPLICAS * len(outs) * width > ws.colacc.numel():
        raise KernelError(f"{len(outs)} column vector(s) of width {width} exceed the shared column workspace "
                          f"({ws.colacc.numel()} floats for {DeferredColumns.REPLICAS} replicas); reduce inside a "
                          "deferred_columns plan instead")
    return ws.colacc, default_counter(ws)


# ----------------------------------------------------------------------------- encoder ops
def embed_ln_fwd(ids, word, pos, gamma, beta, eps, S, p, rng, stream, out, mean, rstd):
    T, H = out.shape
    _call("rb_embed_ln_fwd", _I(DT[out.dtype]), _p(ids), _p(word), _p(pos), _p(gamma), _p(beta), _p(out), _p(mean),
          _p(rstd), _I(T), _I(H), _I(S), _F(eps), _F(p), _p(rng.dev), _U(stream), _stream())


def embed_ln_bwd(dy, ids, word, pos, gamma, mean, rstd, S, p, rng, stream, pad_id, dword, dpos, dgamma, dbeta):
    T, H = dy.shape
    acc, counter = _acc_for([dgamma, dbeta], H, lambda ws: ws.counters)
    dword.zero_()
    dpos.zero_()
    _call("rb_embed_ln_bwd", _I(DT[dy.dtype]), _p(dy), _p(ids), _p(word), _p(pos), _p(gamma), _p(mean), _p(rstd),
          _p(dword), _p(dpos), _p(acc), _p(counter), _p(dgamma), _p(dbeta), _I(T), _I(H), _I(S), _I(pad_id),
          _F(p), _p(rng.dev), _U(stream), _stream())


def _attention_fits(qkv, S: int, H: int, nh: int) -> bool:
    """fp32 activations use the CUDA-core kernels, whose backward tiles exceed shared memory for long
    sequences; those shapes are composed from library ops instead (fp32 encoders are a debugging mode)."""
    if qkv.dtype != torch.float32:
        return S <= 128
    hd = H // nh
    return S <= 128 and 2 * S * (S + 1) * 4 + 4 * S * (hd + 2) * 4 <= 227 * 1024


def _attention_entry(direction: str, H: int, nh: int) -> str:
    """16-bit activations: the register-resident kernels for head dim 64 (scores stay in MMA fragments), the
    shared-memory tile kernels otherwise (head dim 32) or when ``RENEE_B200_ATTENTION=tiles`` asks for them."""
    if H // nh == 64 and os.environ.get("RENEE_B200_ATTENTION", "") != "tiles":
        return f"rb_attention_{direction}_mma"
    return f"rb_attention_{direction}_tc"


def _attention_long(qkv, S: int, H: int, nh: int, ws) -> bool:
    """Sequences of 129..512 tokens, 16-bit activations, head dim 64: the blocked kernels of attention_mma.cu
    (``RENEE_B200_ATTENTION_LONG=0`` sends these shapes to the composed library ops instead)."""
    return (qkv.dtype != torch.float32 and 128 < S <= 512 and H // nh == 64 and "ds" in ws
            and os.environ.get("RENEE_B200_ATTENTION_LONG", "") != "0")


def _seed_tensor(rng):
    # the device-resident seed as a non-negative int64 scalar: no host read, so the composed path can be captured
    return rng.dev.to(torch.int64).reshape(-1)[0] & 0xFFFFFFFF


def attention_fwd(qkv, bqkv, mask, nh, p, rng, stream, ctx_out, ws):
    b, S = mask.shape
    H = ctx_out.shape[1]
    if _attention_long(qkv, S, H, nh, ws):
        _call("rb_attention_fwd_long", _I(DT[qkv.dtype]), _p(qkv), _p(bqkv), _p(mask), _p(ctx_out), _p(ws["probs"]),
              _I(b), _I(S), _I(H), _I(nh), _F(p), _p(rng.dev), _U(stream), _stream())
        return
    if not _attention_fits(qkv, S, H, nh):
        from . import reference as ref
        ctx, probs = ref.attention_fwd(qkv, bqkv, mask, nh, p, _seed_tensor(rng), stream)
        ctx_out.copy_(ctx)
        ws["probs"][:b].copy_(probs)
        return
    _call("rb_attention_fwd" if qkv.dtype == torch.float32 else _attention_entry("fwd", H, nh), _I(DT[qkv.dtype]),
          _p(qkv), _p(bqkv), _p(mask), _p(ctx_out), _p(ws["probs"]), _I(b), _I(S),
          _I(H), _I(nh), _F(p), _p(rng.dev), _U(stream), _stream())


def attention_bwd(dctx, qkv, bqkv, mask, nh, p, rng, stream, ws, dqkv_out, dbqkv_out):
    b, S = mask.shape
    H = dctx.shape[1]
    if _attention_long(qkv, S, H, nh, ws):
        acc = _DEFER.slot([dbqkv_out], 3 * H) if _DEFER is not None else None
        _call("rb_attention_bwd_long", _I(DT[qkv.dtype]), _p(dctx), _p(qkv), _p(bqkv), _p(ws["probs"]), _p(ws["ds"]),
              _p(dqkv_out), _I(b), _I(S), _I(H), _I(nh), _F(p), _p(rng.dev), _U(stream), _p(acc), _stream(), launches=2)
        if acc is None:
            colsum(dqkv_out, dbqkv_out)
        return
    if not _attention_fits(qkv, S, H, nh):
        from . import reference as ref
        d = ref.attention_bwd(dctx, qkv, bqkv, mask, ws["probs"][:b], nh, p, _seed_tensor(rng), stream)
        dqkv_out.copy_(d)
        colsum(dqkv_out, dbqkv_out)
        return
    if qkv.dtype == torch.float32:
        _call("rb_attention_bwd", _I(DT[qkv.dtype]), _p(dctx), _p(qkv), _p(bqkv), _p(ws["probs"]), _p(dqkv_out), _I(b),
              _I(S), _I(H), _I(nh), _F(p), _p(rng.dev), _U(stream), _stream())
        colsum(dqkv_out, dbqkv_out)
        return
    # with a deferred-columns plan active the kernel also accumulates the q/k/v bias gradients
    acc = _DEFER.slot([dbqkv_out], 3 * H) if _DEFER is not None else None
    _call(_attention_entry("bwd", H, nh), _I(DT[qkv.dtype]), _p(dctx), _p(qkv), _p(bqkv), _p(ws["probs"]), _p(dqkv_out), _I(b),
          _I(S), _I(H), _I(nh), _F(p), _p(rng.dev), _U(stream), _p(acc), _stream())
    if acc is None:
        colsum(dqkv_out, dbqkv_out)


def bias_dropout_add_ln_fwd(x, bias, resid, gamma, beta, eps, p, rng, stream, y_out, pre_out, mean, rstd):
    T, H = x.shape
    _call("rb_bias_dropout_add_ln_fwd", _I(DT[x.dtype]), _p(x), _p(bias), _p(resid), _p(gamma), _p(beta), _p(y_out),
          _p(pre_out), _p(mean), _p(rstd), _I(T), _I(H), _F(eps), _F(p), _p(rng.dev), _U(stream), _stream())


def bias_dropout_add_ln_bwd(dy, pre, gamma, mean, rstd, p, rng, stream, dgamma, dbeta, dbias, dpre_out, dbranch_out):
    T, H = dy.shape
    acc, counter = _acc_for([dgamma, dbeta, dbias], H, lambda ws: ws.counters)
    _call("rb_bias_dropout_add_ln_bwd", _I(DT[dy.dtype]), _p(dy), _p(pre), _p(gamma), _p(mean), _p(rstd), _p(dpre_out),
          _p(dbranch_out if p > 0 else None), _p(acc), _p(counter), _p(dgamma), _p(dbeta), _p(dbias),
          _I(T), _I(H), _F(p), _p(rng.dev), _U(stream), _stream())
    return (dpre_out, dbranch_out) if p > 0 else (dpre_out, dpre_out)


def bias_gelu_fwd(x, bias, out):
    T, Fd = x.shape
    _call("rb_bias_gelu_fwd", _I(DT[x.dtype]), _p(x), _p(bias), _p(out), _I(T), _I(Fd), _stream())


def bias_gelu_bwd(da, x, bias, dbias, dx_out):
    T, Fd = x.shape
    acc, counter = _acc_for([dbias], Fd, lambda ws: ws.counters[1:])
    _call("rb_bias_gelu_bwd", _I(DT[x.dtype]), _p(da), _p(x), _p(bias), _p(dx_out), _p(acc), _p(counter),
          _p(dbias), _I(T), _I(Fd), _stream())


# ----------------------------------------------------------------------------- encoder GEMMs (tcgen05, fused epilogues)
L_NT, L_NN, L_TN = 0, 1, 2
E_STORE, E_BIAS_GELU, E_BIAS_DROPOUT_RESID, E_ADD, E_GELU_BWD, E_SPLITK = 0, 1, 2, 3, 4, 5


class _SplitKScratch:
    """fp32 partial-sum tiles and per-tile arrival counters of the split-K weight-gradient GEMMs.  Both are zero
    between launches by contract of the kernel (the last CTA of a tile re-zeroes what it consumed).  Grows on
    demand, so the shapes of a training step must have been seen once before the step is captured in a graph."""

    def __init__(self):
        self.buf = None
        self.counters = None

    def get(self, device, floats: int, tiles: int):
        if self.buf is None or self.buf.numel() < floats:
            self.buf = torch.zeros(floats, dtype=torch.float32, device=device)
        if self.counters is None or self.counters.numel() < tiles:
            self.counters = torch.zeros(max(tiles, 256), dtype=torch.int32, device=device)
        return self.buf, self.counters


_SK: dict = {}


def enc_gemm_supported(t: torch.Tensor, *dims: int) -> bool:
    """The own GEMMs serve 16-bit CUDA tensors whose feature dimensions are multiples of 64."""
    return bool(t.is_cuda and t.dtype in (torch.bfloat16, torch.float16) and all(d % 64 == 0 for d in dims)
                and os.environ.get("RENEE_B200_OWN_GEMM", "auto") != "0")


def _enc_gemm(layout, epi, A, B, C, M, N, K, bias=None, R=None, F=None, p=0.0, rng=None, stream=0, colacc=None,
              col_tot=0, col_off=0, bn=0, ncta=0):
    dev = C.device
    ws = workspace(dev)
    sk_buf, sk_cnt = None, None
    if not bn:
        bn = int(os.environ.get("RENEE_B200_GEMM_BN", "0"))        # experiments: force the N tile / the tile shape
    if not ncta:
        ncta = int(os.environ.get("RENEE_B200_GEMM_NCTA", "0"))
    if layout == L_TN:
        ncta_o, bn_o, sp_o, words_o, floats_o = _I(0), _I(0), _I(0), _I(0), _LL(0)
        lib().rb_enc_gemm_plan(_I(layout), _I(epi), _I(M), _I(N), _I(K), _I(bn), _I(ncta), _c.byref(ncta_o), _c.byref(bn_o),
                               _c.byref(sp_o), _c.byref(floats_o), _c.byref(words_o))
        if sp_o.value > 1:
            key = dev.index if dev.index is not None else torch.cuda.current_device()
            sk_buf, sk_cnt = _SK.setdefault(key, _SplitKScratch()).get(dev, floats_o.value, words_o.value)
    _call("rb_enc_gemm", _I(DT[C.dtype]), _I(layout), _I(epi), _p(A), _p(B), _p(C), _I(M), _I(N), _I(K),
          _I(A.stride(0)), _I(B.stride(0)), _I(C.stride(0)), _p(bias), _p(R), _I(R.stride(0) if R is not None else 0),
          _p(F), _I(F.stride(0) if F is not None else 0), _F(p), _p(rng.dev if rng is not None else None), _U(stream),
          _p(colacc), _I(col_tot), _I(col_off), _p(sk_buf), _p(sk_cnt), _I(bn), _I(ncta), _p(ws.status), _stream())


def linear_fwd(x, W, out, epi="store", bias=None, resid=None, pre_out=None, p=0.0, rng=None, stream=0, bn=0, ncta=0):
    """``out = epilogue(x @ W.T)`` for ``x [T, K]``, ``W [N, K]`` (an ``nn.Linear`` weight):

    * ``store``: the product;
    * ``bias_gelu``: ``pre_out = x W^T + bias`` (kept for the backward pass), ``out = gelu(pre_out)``;
    * ``bias_dropout_resid``: ``out = resid + dropout(x W^T + bias)`` — the input of the following LayerNorm.

    ``bn`` / ``ncta`` force the N tile (64, 128, 256) and the tile shape (1: one CTA per 128-row tile, 2: a CTA
    pair per 256-row tile); 0 lets the library choose."""
    T, K = x.shape
    N = W.shape[0]
    code = {"store": E_STORE, "bias_gelu": E_BIAS_GELU, "bias_dropout_resid": E_BIAS_DROPOUT_RESID}[epi]
    _enc_gemm(L_NT, code, x, W, out, T, N, K, bias=bias, R=resid, F=pre_out, p=p, rng=rng, stream=stream, bn=bn, ncta=ncta)
    return out


def linear_dgrad(dy, W, out, epi="store", resid=None, pre=None, dbias=None, bn=0, ncta=0):
    """``out = epilogue(dy @ W)`` for ``dy [T, N]``, ``W [N, K]``:

    * ``store``: the product;  ``add``: product ``+ resid`` (the residual branch's gradient);
    * ``gelu_bwd``: product ``* gelu'(pre)`` with ``pre`` the stored pre-activation, and its column sums written
      to ``dbias`` (through the active deferred-column plan, or at once when there is none)."""
    T, N = dy.shape
    K = W.shape[1]
    code = {"store": E_STORE, "add": E_ADD, "gelu_bwd": E_GELU_BWD}[epi]
    if code != E_GELU_BWD or dbias is None:
        _enc_gemm(L_NN, code, dy, W, out, T, K, N, R=resid if code == E_ADD else pre, bn=bn, ncta=ncta)
        return out
    plan = _DEFER if _DEFER is not None else DeferredColumns(out.device, out.dtype)
    acc = plan.slot([dbias], K)
    _enc_gemm(L_NN, code, dy, W, out, T, K, N, R=pre, colacc=acc, col_tot=K, col_off=0, bn=bn, ncta=ncta)
    if _DEFER is None:
        plan.finalize()
    return out


def linear_wgrad(dy, x, dW, bn=0, ncta=0):
    """``dW = dy.T @ x`` for ``dy [T, N]``, ``x [T, K]``, ``dW [N, K]`` (split over T, reduced in fp32)."""
    T, N = dy.shape
    K = x.shape[1]
    _enc_gemm(L_TN, E_SPLITK, dy, x, dW, N, K, T, bn=bn, ncta=ncta)
    return dW


def ln_fwd(pre, gamma, beta, eps, y_out, mean, rstd):
    T, H = pre.shape
    _call("rb_ln_fwd", _I(DT[pre.dtype]), _p(pre), _p(gamma), _p(beta), _p(y_out), _p(mean), _p(rstd), _I(T), _I(H),
          _F(eps), _stream())


def colsum(x, out):
    T, N = x.shape
    acc, counter = _acc_for([out], N, lambda ws: ws.counters[2:])
    _call("rb_colsum", _I(DT[x.dtype]), _p(x), _p(acc), _p(counter), _p(out), _I(T), _I(N), _stream())
    return out


def pool_fwd(h, mask, mode, out):
    b, S, H = h.shape
    _call("rb_pool_fwd", _I(DT[h.dtype]), _p(h), _p(mask), _p(out), _I(b), _I(S), _I(H), _I(1 if mode == "cls" else 0),
          _stream())


def pool_bwd(de, mask, mode, S, dh_out):
    b, H = de.shape
    _call("rb_pool_bwd", _I(DT[dh_out.dtype]), _p(de), _p(mask), _p(dh_out), _I(b), _I(S), _I(H),
          _I(1 if mode == "cls" else 0), _stream())


def dropout_cast_fwd(e, p, rng, stream, out):
    _call("rb_dropout_cast_fwd", _I(DT[out.dtype]), _p(e), _p(out), _LL(e.numel()), _F(p), _p(rng.dev), _U(stream),
          _stream())


def dropout_bwd(dx, p, rng, stream, out):
    _call("rb_dropout_cast_fwd", _I(DT[out.dtype]), _p(dx), _p(out), _LL(dx.numel()), _F(p), _p(rng.dev), _U(stream),
          _stream())


# ----------------------------------------------------------------------------- optimizer
def grad_check(g, hp):
    _call("rb_grad_check", _I(DT[g.dtype]), _p(g), _LL(g.numel()), _p(hp.buf), _stream())


def adamw_step(p32, m, v, g, p16, hp, beta1, beta2, eps, wd, n_decay, grad_mult: float = 1.0):
    _call("rb_adamw", _I(DT[g.dtype]), _p(p32), _p(m), _p(v), _p(g), _p(None if p16 is p32 else p16), _LL(p32.numel()),
          _LL(n_decay), _p(hp.buf), _F(beta1), _F(beta2), _F(eps), _F(wd), _F(grad_mult), _stream())


def scaler_update(buf, enabled, growth, backoff, interval):
    _call("rb_scaler_update", _p(buf), _I(1 if enabled else 0), _F(growth), _F(backoff), _I(interval), _stream())


# ----------------------------------------------------------------------------- classifier step
def _ld_g(B: int) -> int:
    return (B + 7) // 8 * 8


def xfc_logits_grad(W, X, Gt, ldG, pos_rows, pos_labels, nnz, label0, loss_acc=None, raw_out=None, wait=None):
    """``wait = (flags_tensor, n, step_tensor)``: the producer warp waits until ``flags[0:n] >= *step``
    (the all-gather of X has landed) before its first load."""
    Lc, D = W.shape
    B = X.shape[0]
    ws = workspace(W.device)
    wf, wn, wstep = (wait if wait is not None else (None, 0, None))
    _call("rb_xfc_logits_grad", _p(W), _I(Lc), _I(D), _p(X), _I(B), _p(Gt), _I(ldG), _p(pos_rows), _p(pos_labels),
          _p(nnz), _I(label0), _p(loss_acc), _p(raw_out), _p(wf), _I(wn), _p(wstep), _p(ws.status), _stream())


def xfc_v2() -> bool:
    """The classifier's logits+gradient and dX GEMMs run on the persistent CTA-pair GEMM of ``gemm.cu`` (positives
    applied to the staged tile in shared memory, dX by scaled vector reductions); ``RENEE_B200_XFC_V2=0`` selects the
    one-tile-per-CTA kernels of ``xfc.cu`` instead.  Steps that sample the loss always use the latter (its epilogue
    carries the loss partial sums)."""
    return os.environ.get("RENEE_B200_XFC_V2", "1") != "0"


def xfc_logits_grad_v2(W, X, Gt, ldG, pos_rows, pos_labels, nnz, label0, wait=None, loss_acc=None):
    """``Gt = sigmoid(W Xᵀ) - Y`` on the persistent CTA-pair GEMM; with ``loss_acc`` also ``+= Σ softplus(z)``."""
    Lc, D = W.shape
    B = X.shape[0]
    ws = workspace(W.device)
    wf, wn, wstep = (wait if wait is not None else (None, 0, None))
    _call("rb_xfc_logits_grad_v2", _p(W), _I(Lc), _I(D), _p(X), _I(B), _p(Gt), _I(ldG), _p(pos_rows), _p(pos_labels), _p(nnz),
          _I(label0), _p(wf), _I(wn), _p(wstep), _p(loss_acc), _p(ws.status), _stream())


def xfc_dx_v2(Gt, ldG, W, B, dX, hp_buf, signal=None):
    Lc, D = W.shape
    ws = workspace(W.device)
    if signal is None:
        cnt, ptrs, n, idx, step = None, None, 0, 0, None
    else:
        cnt, ptrs, n, idx, step = signal
    _call("rb_xfc_dx_v2", _p(Gt), _I(ldG), _p(W), _I(Lc), _I(D), _I(B), _p(dX), _p(hp_buf), _p(cnt),
          ptrs if ptrs is not None else _VP(0), _I(n), _I(idx), _p(step), _p(ws.status), _stream())


def set_xfc_persistent(on: bool) -> None:
    """Chooses the persistent logits kernel (one CTA per SM walking the tiles, epilogue of tile i under the main
    loop of tile i + 1) for label chunks with more 128-label tiles than SMs.  Off by default."""
    lib().rb_xfc_set_persistent(_I(1 if on else 0))


def xfc_dx(Gt, ldG, W, B, dX, hp_buf, splits, signal=None):
    """``signal = (counter_tensor, peer_flag_ptr_array, n_peers, flag_index, step_tensor)``: the last CTA
    stores ``*step`` into word ``flag_index`` of every peer's flag array (reduce-scatter signal)."""
    Lc, D = W.shape
    ws = workspace(W.device)
    if signal is None:
        cnt, ptrs, n, idx, step = None, None, 0, 0, None
    else:
        cnt, ptrs, n, idx, step = signal
    _call("rb_xfc_dx", _p(Gt), _I(ldG), _p(W), _I(Lc), _I(D), _I(B), _p(dX), _p(hp_buf), _I(splits), _p(cnt),
          ptrs if ptrs is not None else _VP(0), _I(n), _I(idx), _p(step), _p(ws.status), _stream())


def xfc_dw_sgd(Gt, ldG, X, W, M, hp_buf, mo, wd, tma_tiles=True, stochastic_round=False, v2=False, bn=0, ncta=0):
    """W, M updated in place from dW = Gt X (never stored).  ``v2``: the persistent CTA-pair GEMM with the W / M tiles
    staged through shared memory by TMA; otherwise the one-tile-per-CTA kernel."""
    Lc, D = W.shape
    B = X.shape[0]
    ws = workspace(W.device)
    if v2:
        _call("rb_xfc_dw_sgd_v2", _p(Gt), _I(ldG), _p(X), _I(B), _p(W), _p(M), _I(Lc), _I(D), _p(hp_buf), _F(mo), _F(wd),
              _I(1 if stochastic_round else 0), _I(bn), _I(ncta), _p(ws.status), _stream())
        return
    _call("rb_xfc_dw_sgd", _p(Gt), _I(ldG), _p(X), _I(B), _p(W), _p(M), _I(Lc), _I(D), _p(hp_buf), _F(mo), _F(wd),
          _I(int(tma_tiles)), _I(1 if stochastic_round else 0), _p(ws.status), _stream())


_SMS: dict = {}


def sm_count(device=None) -> int:
    """Number of SMs of ``device`` (the current one by default), queried once."""
    idx = torch.device(device).index if device is not None and torch.device(device).index is not None \
        else torch.cuda.current_device()
    if idx not in _SMS:
        _SMS[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return _SMS[idx]


def dx_splits(B: int, D: int, Lc: int) -> int:
    """Split-K factor of the dX GEMM so that the grid covers the SMs about once."""
    tiles = ((B + 127) // 128) * ((D + 255) // 256)
    kb = (Lc + 63) // 64
    sms = sm_count()
    return max(1, min(kb, (sms + tiles - 1) // tiles))


def xfc_step(xfc, X, pos_rows, pos_labels, nnz, dX_out, hp, mo, wd, want_loss, wait=None, signal=None,
             side_stream=None):
    """Chunked K1 → K3 → K2 over the label shard (see :class:`renee_b200.models.xfc.XFCClassifier`).
    ``wait`` is handed to the first logits GEMM (all-gather prologue), ``signal`` to the last dX GEMM
    (reduce-scatter epilogue).  With ``side_stream`` the last chunk's dW+SGD kernel — HBM-bound, and
    nothing downstream in this step depends on it — is issued on that stream so that it overlaps the
    compute-bound encoder backward; the caller joins the stream before the step ends."""
    B, D = X.shape
    ldG = _ld_g(B)
    sc = xfc.scratch(B)
    Gt = sc["Gt"]
    loss = None
    if want_loss:
        loss = sc.setdefault("loss", torch.zeros(1, dtype=torch.float32, device=X.device))
        loss.zero_()
    dX_out.zero_()
    chunks = list(range(0, xfc.Ls, xfc.chunk))
    dw_v2 = xfc_v2() and os.environ.get("RENEE_B200_XFC_DW_V2", "1") != "0"
    for ci, l0 in enumerate(chunks):
        l1 = min(xfc.Ls, l0 + xfc.chunk)
        Wc, Mc = xfc.W[l0:l1], xfc.M[l0:l1]
        v2 = xfc_v2() and D % 64 == 0
        if v2:
            xfc_logits_grad_v2(Wc, X, Gt, ldG, pos_rows, pos_labels, nnz, l0, wait=wait if ci == 0 else None,
                               loss_acc=loss)
        else:
            xfc_logits_grad(Wc, X, Gt, ldG, pos_rows, pos_labels, nnz, l0, loss_acc=loss, wait=wait if ci == 0 else None)
        if want_loss and ci == 0:
            # minus the logits at the positives, taken before any chunk's weights are updated (and after
            # the first GEMM's wait, so X is complete)
            _call("rb_xfc_pos_logit_sum", _p(xfc.W), _p(X), _I(D), _p(pos_rows), _p(pos_labels), _p(nnz), _p(loss),
                  _stream())
        if v2:
            xfc_dx_v2(Gt, ldG, Wc, B, dX_out, hp.buf, signal=signal if ci == len(chunks) - 1 else None)
        else:
            xfc_dx(Gt, ldG, Wc, B, dX_out, hp.buf, dx_splits(B, D, l1 - l0), signal=signal if ci == len(chunks) - 1 else None)
        if side_stream is not None and ci == len(chunks) - 1:
            main = torch.cuda.current_stream()
            side_stream.wait_stream(main)
            with torch.cuda.stream(side_stream):
                xfc_dw_sgd(Gt, ldG, X, Wc, Mc, hp.buf, mo, wd, stochastic_round=xfc.stochastic_round, v2=dw_v2)
        else:
            xfc_dw_sgd(Gt, ldG, X, Wc, Mc, hp.buf, mo, wd, stochastic_round=xfc.stochastic_round, v2=dw_v2)
    return loss[0] if want_loss else None


def topk_rows(Z, n, k, label0, out_val, out_idx):
    """Unordered top-k of each row of batch-major fp32 logits ``Z[B, ldZ]`` (first ``n`` columns valid)."""
    B, ldZ = Z.shape
    _call("rb_topk_rows", _p(Z), _I(ldZ), _I(B), _I(n), _I(k), _I(label0), _p(out_val), _p(out_idx), _stream())


def xfc_topk8(W, X, k):
    """Top-k (k <= 8) of every row of ``X Wᵀ`` with the selection fused into the GEMM epilogue: each epilogue
    thread of the persistent tcgen05 GEMM keeps the 8 best entries of its row over all label tiles its CTA
    visits, so the ``[B, Ls]`` logits are never written; the few thousand candidates per row are then reduced by
    the row-selection kernel.  Returns ``(values [B, k] fp32 descending, label ids [B, k] int64)``."""
    B, D = X.shape
    Ls = W.shape[0]
    width = int(lib().rb_xfc_topk8_width())
    cv = torch.full((B, width), -3.0e38, dtype=torch.float32, device=X.device)
    ci = torch.zeros(B, width, dtype=torch.int32, device=X.device)
    ws = workspace(X.device)
    _call("rb_xfc_topk8", _I(DT[X.dtype]), _p(X), _p(W), _I(B), _I(Ls), _I(D), _I(X.stride(0)), _I(W.stride(0)), _p(cv),
          _p(ci), _I(width), _p(ws.status), _stream())
    vals = torch.empty(B, k, dtype=torch.float32, device=X.device)
    pos = torch.empty(B, k, dtype=torch.int32, device=X.device)
    topk_rows(cv, width, k, 0, vals, pos)
    idx = torch.gather(ci, 1, pos.long())
    v, order = torch.sort(vals, dim=1, descending=True)
    return v, torch.gather(idx, 1, order).long()


def xfc_topk(xfc, X, k):
    """Local top-k of ``X Wᵀ`` over this rank's shard.  ``k <= 8`` (evaluation during training uses 5): fused into
    the GEMM epilogue (:func:`xfc_topk8`).  Larger ``k`` (100 for the final evaluation): per label chunk, the tcgen05
    logits GEMM writes fp32 logits batch-major into an L2-sized buffer and a radix-select kernel extracts each
    row's k best; the per-chunk candidates (k each) are merged at the end."""
    B, D = X.shape
    k_eff = min(k, xfc.Ls)
    if k_eff <= 8 and D % 64 == 0 and os.environ.get("RENEE_B200_FUSED_TOPK", "1") != "0":
        return xfc_topk8(xfc.W, X, k_eff)
    chunk = min(xfc.chunk, max(128, (32 << 20) // (4 * B) // 128 * 128))
    ldZ = (min(chunk, xfc.Ls) + 7) // 8 * 8
    Z = torch.empty(B, ldZ, dtype=torch.float32, device=X.device)
    starts = list(range(0, xfc.Ls, chunk))
    vals = torch.empty(len(starts), B, k_eff, dtype=torch.float32, device=X.device)
    idxs = torch.empty(len(starts), B, k_eff, dtype=torch.int32, device=X.device)
    for ci, l0 in enumerate(starts):
        l1 = min(xfc.Ls, l0 + chunk)
        xfc_logits_grad(xfc.W[l0:l1], X, None, ldZ, None, None, None, l0, raw_out=Z)
        topk_rows(Z, l1 - l0, k_eff, l0, vals[ci], idxs[ci])
    cv = vals.permute(1, 0, 2).reshape(B, -1)
    ci_ = idxs.permute(1, 0, 2).reshape(B, -1)
    v, sel = torch.topk(cv, k_eff, dim=1)
    return v, torch.gather(ci_, 1, sel).long()


# ----------------------------------------------------------------------------- peer-memory collectives
class _RawCudaBuffer:
    """Device memory obtained from ``cudaMalloc`` by this library, exposed through
    ``__cuda_array_interface__`` so that PyTorch can view it without owning it."""

    def __init__(self, ptr: int, nbytes: int):
        self.ptr, self.nbytes = int(ptr), int(nbytes)
        self.__cuda_array_interface__ = {"shape": (self.nbytes,), "typestr": "|u1", "data": (self.ptr, False),
                                         "version": 2, "strides": None}


def ipc_alloc(numel: int, dtype, device) -> torch.Tensor:
    """A zero-filled tensor in its own ``cudaMalloc`` allocation (exportable with :func:`ipc_export`).  The
    allocation lives until the process exits."""
    esz = torch.empty((), dtype=dtype).element_size()
    nbytes = (numel * esz + 255) // 256 * 256
    out = _VP(0)
    with torch.cuda.device(device):
        rc = lib().rb_ipc_alloc(_LL(nbytes), _c.byref(out))
    if rc != 0:
        raise KernelError(f"rb_ipc_alloc({nbytes}) failed with CUDA error {rc}")
    raw = torch.as_tensor(_RawCudaBuffer(out.value, nbytes), device=device)
    return raw.view(dtype)[:numel]


def ipc_export(t: torch.Tensor) -> bytes:
    """CUDA IPC handle of the allocation ``t`` starts at (``t`` must come from :func:`ipc_alloc`)."""
    n = lib().rb_ipc_handle_bytes()
    buf = _c.create_string_buffer(n)
    rc = lib().rb_ipc_export(_VP(t.data_ptr()), buf)
    if rc != 0:
        raise KernelError(f"cudaIpcGetMemHandle failed with CUDA error {rc}")
    return bytes(buf.raw)


def ipc_open(handle: bytes, device) -> int:
    """Maps another process's allocation into this process (peer access enabled on demand); returns its
    device address."""
    out = _VP(0)
    with torch.cuda.device(device):
        rc = lib().rb_ipc_open(_c.c_char_p(handle), _c.byref(out))
    if rc != 0:
        raise KernelError(f"cudaIpcOpenMemHandle failed with CUDA error {rc}")
    return int(out.value)


def ptr_array(ptrs):
    """ctypes ``void*[n]`` from a list of integer device addresses (kept alive by the caller)."""
    return (_VP * len(ptrs))(*[_VP(int(x)) for x in ptrs])


def step_inc(step):
    _call("rb_step_inc", _p(step), _stream())


def ag_push(e, p, rng, stream_id, xbuf_ptrs, row0, flag_ptrs, flag_base, my_rank, G, step, counters):
    b, D = e.shape
    _call("rb_ag_push", _p(e), _I(b), _I(D), _F(p), _p(rng.dev), _U(stream_id), xbuf_ptrs, _I(row0), flag_ptrs,
          _I(flag_base), _I(my_rank), _I(G), _p(step), _p(counters), _stream())


def peer_gather(src, dst_ptrs, slot_bytes, flag_ptrs, flag_base, my_rank, G, step, counters):
    """Copies ``src`` (contiguous, a multiple of 16 bytes) into every rank's buffer at byte offset ``slot_bytes`` and
    raises this rank's flag of class ``flag_base`` there."""
    nbytes = src.numel() * src.element_size()
    _call("rb_peer_gather", _p(src), _LL(nbytes), dst_ptrs, _LL(slot_bytes), flag_ptrs, _I(flag_base), _I(my_rank), _I(G),
          _p(step), _p(counters), _stream())


def rs_pull(partial_ptrs, G, row0, b, D, de, my_flags, step, p, rng, stream_id):
    ws = workspace(de.device)
    _call("rb_rs_pull", partial_ptrs, _I(G), _I(row0), _I(b), _I(D), _p(de), _p(my_flags), _p(step), _F(p), _p(rng.dev),
          _U(stream_id), _p(ws.status), _stream())


def signal(flag_ptrs, G, flag_base, my_rank, step, mul=1, add=0):
    _call("rb_signal", flag_ptrs, _I(G), _I(flag_base), _I(my_rank), _p(step), _U(mul), _U(add), _stream())


def wait_flags(my_flags, G, step, mul=1, add=0, found_words=None, hp_buf=None):
    ws = workspace(my_flags.device)
    _call("rb_wait_flags", _p(my_flags), _I(G), _p(step), _U(mul), _U(add), _p(found_words), _p(hp_buf), _p(ws.status),
          _stream())


def grad_allreduce(g_dtype, grad_ptrs, lo, hi, G, my_rank, my_flags_a, flag_ptrs, flag_b_base, found_base, step, mul, add,
                   counter, blocks):
    ws = workspace(my_flags_a.device)
    _call("rb_grad_allreduce", _I(DT[g_dtype]), grad_ptrs, _LL(lo), _LL(hi), _I(G), _I(my_rank), _p(my_flags_a), flag_ptrs,
          _I(flag_b_base), _I(found_base), _p(step), _U(mul), _U(add), _p(counter), _I(blocks), _p(ws.status), _stream())


def grad_reduce_scatter(g_dtype, grad_ptrs, n, G, my_rank, my_flags_a, step, gsum, flag_ptrs, flag_b_base, found_base,
                        counter, blocks, mc_grads: int = 0):
    ws = workspace(my_flags_a.device)
    _call("rb_grad_reduce_scatter", _I(DT[g_dtype]), grad_ptrs, _LL(n), _I(G), _I(my_rank), _p(my_flags_a), _p(step),
          _p(gsum), flag_ptrs, _I(flag_b_base), _I(found_base), _p(counter), _I(blocks), _p(ws.status), _VP(mc_grads),
          _stream())


def grad_reduce_scatter_range(g_dtype, grad_ptrs, v0, v1, G, my_rank, my_flags_a, step, mul_a, add_a, gsum, flag_ptrs,
                              flag_b_base, found_base, counter, blocks, mc_grads: int = 0):
    """Sums vectors ``[v0, v1)`` (8 elements each) of the flat gradient over all ranks into ``gsum``; waits until
    every rank's progress flag has reached ``step * mul_a + add_a``; ``flag_b_base < 0``: no completion signal."""
    ws = workspace(my_flags_a.device)
    _call("rb_grad_reduce_scatter_range", _I(DT[g_dtype]), grad_ptrs, _LL(v0), _LL(v1), _I(G), _I(my_rank), _p(my_flags_a),
          _p(step), _U(mul_a), _U(add_a), _p(gsum), flag_ptrs, _I(flag_b_base), _I(found_base), _p(counter), _I(blocks),
          _p(ws.status), _VP(mc_grads), _stream())


def adamw_ranges_push(p_dtype, p32, m, v, gsum, p16_ptrs, ranges, n_decay, G, my_rank, hp_buf, beta1, beta2, eps, wd,
                      grad_mult, flag_ptrs, flag_c_base, step, counter, blocks, mc_p16: int = 0):
    """AdamW on ``ranges = [(v0, v1, g0), ...]`` (vector ranges of the flat buffer, start of their sums in ``gsum``)
    and the push of the updated 16-bit values into every rank's compute copy."""
    n = len(ranges)
    arr = _LL * max(n, 1)
    v0, v1, g0 = arr(*[r[0] for r in ranges]), arr(*[r[1] for r in ranges]), arr(*[r[2] for r in ranges])
    _call("rb_adamw_ranges_push", _I(DT[p_dtype]), _p(p32), _p(m), _p(v), _p(gsum), p16_ptrs, _I(n), v0, v1, g0,
          _LL(n_decay), _I(G), _I(my_rank), _p(hp_buf), _F(beta1), _F(beta2), _F(eps), _F(wd), _F(grad_mult), flag_ptrs,
          _I(flag_c_base), _p(step), _p(counter), _I(blocks), _VP(mc_p16), _stream())


def adamw_shard_push(p_dtype, p32, m, v, gsum, p16_ptrs, n, n_decay, G, my_rank, hp_buf, beta1, beta2, eps, wd, grad_mult,
                     flag_ptrs, flag_c_base, step, counter, blocks, mc_p16: int = 0):
    _call("rb_adamw_shard_push", _I(DT[p_dtype]), _p(p32), _p(m), _p(v), _p(gsum), p16_ptrs, _LL(n), _LL(n_decay), _I(G),
          _I(my_rank), _p(hp_buf), _F(beta1), _F(beta2), _F(eps), _F(wd), _F(grad_mult), flag_ptrs, _I(flag_c_base),
          _p(step), _p(counter), _I(blocks), _VP(mc_p16), _stream())
