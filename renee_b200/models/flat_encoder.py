"""Flat-buffer encoder engine with a hand-written forward and backward pass.

The reference runs the HF encoder under autograd, DDP and apex FusedAdam (main.py:160-161,
177-181; dl_base.py:299-300, 360, 372).  On B200 the 131K-label configurations are launch-bound,
so this engine is built for CUDA-graph capture instead:

* every parameter is a view into ONE flat fp32 master buffer (decayed parameters first, then the
  no-decay group), with a low-precision compute copy, a flat gradient buffer and flat Adam moments —
  the gradient all-reduce and the fused AdamW each touch one contiguous range;
* the q/k/v projections are adjacent in the buffer, so one GEMM computes all three;
* forward and backward are explicit sequences of GEMMs and fused kernels from :mod:`renee_b200.ops`
  (attention, LayerNorm, embedding gather+LayerNorm, pooling), writing into pre-allocated activations;
  no autograd graph, no allocator calls inside the step.  With 16-bit activations on a GPU every
  linear layer is an own tcgen05 GEMM (``ops/csrc/gemm.cu``) whose epilogue carries its element-wise
  neighbours: bias + GELU (storing the pre-activation), bias + dropout + residual (producing the
  LayerNorm input), GELU backward + bias-gradient column sums, the residual-gradient add of the
  data-gradient GEMMs, and a split-K weight-gradient GEMM.  fp32 activations (CPU, debugging mode) use
  library GEMMs and stand-alone element-wise ops;
* dropout masks are recomputed from a counter-based RNG in the backward pass.

State-dict keys are those of HF DistilBERT (see :mod:`renee_b200.models.encoder`).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass

import torch

from .. import ops
from ..utils import guard
from .encoder import EncoderConfig

ALIGN = 128  # elements; keeps every parameter 256-byte aligned in bf16


# dropout stream ids (call sites); layer l uses base + 8*l
_S_EMB, _S_ATTN, _S_FFN, _S_PROBS, _S_CLS = 1, 2, 3, 4, 5


def _no_decay(name: str) -> bool:
    """The reference's no-decay filter is a substring match on ``bias``, ``LayerNorm.bias`` and
    ``LayerNorm.weight`` (dl_base.py:229).  DistilBERT names its block norms ``sa_layer_norm`` /
    ``output_layer_norm``, so only biases and ``embeddings.LayerNorm.weight`` escape weight decay."""
    return any(nd in name for nd in ("bias", "LayerNorm.bias", "LayerNorm.weight"))


# Tokens per step and GPU from which the own GEMMs are used in "auto" mode.  Measured step times on one B200, own /
# library GEMMs: 16384 tokens 7.14 / 7.12 ms, 8192: 3.76 / 3.61, 4096: 2.41 / 2.23, 2048: 1.82 / 1.53, 1024: 1.48 /
# 1.22 -- below 8192 tokens the fixed cost per launch of a persistent kernel (TMEM allocation, cluster start-up, a
# serial K loop on the few SMs the tiles cover) outweighs the fused epilogues.
OWN_GEMM_MIN_TOKENS = int(os.environ.get("RENEE_B200_OWN_GEMM_MIN_TOKENS", "8192"))


@dataclass
class _Slot:
    offset: int
    shape: tuple
    numel: int


class FlatEncoder:
    def __init__(self, cfg: EncoderConfig, device, act_dtype=torch.bfloat16, pooling: str = "mean",
                 bottleneck_dims: int = 0, seed: int = 0, grad_alloc=None, p16_alloc=None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.act_dtype = act_dtype
        self.pooling = pooling
        self.bottleneck_dims = int(bottleneck_dims)
        self.out_dims = self.bottleneck_dims if self.bottleneck_dims > 0 else cfg.dim
        H, Fd = cfg.dim, cfg.hidden_dim
        names = [("embeddings.word_embeddings.weight", (cfg.vocab_size, H)),
                 ("embeddings.position_embeddings.weight", (cfg.max_position_embeddings, H)),
                 ("embeddings.LayerNorm.weight", (H,)), ("embeddings.LayerNorm.bias", (H,))]
        for l in range(cfg.n_layers):
            p = f"transformer.layer.{l}."
            names += [(p + "attention.q_lin.weight", (H, H)), (p + "attention.k_lin.weight", (H, H)),
                      (p + "attention.v_lin.weight", (H, H)),
                      (p + "attention.q_lin.bias", (H,)), (p + "attention.k_lin.bias", (H,)),
                      (p + "attention.v_lin.bias", (H,)),
                      (p + "attention.out_lin.weight", (H, H)), (p + "attention.out_lin.bias", (H,)),
                      (p + "sa_layer_norm.weight", (H,)), (p + "sa_layer_norm.bias", (H,)),
                      (p + "ffn.lin1.weight", (Fd, H)), (p + "ffn.lin1.bias", (Fd,)),
                      (p + "ffn.lin2.weight", (H, Fd)), (p + "ffn.lin2.bias", (H,)),
                      (p + "output_layer_norm.weight", (H,)), (p + "output_layer_norm.bias", (H,))]
        self.encoder_param_names = [n for n, _ in names]
        if self.bottleneck_dims > 0:
            names.append(("__bottleneck__.transformer_weight", (self.bottleneck_dims, H)))
        decay = [(n, s) for n, s in names if not _no_decay(n)]
        nodecay = [(n, s) for n, s in names if _no_decay(n)]
        # the (decayed) block LayerNorm weights go behind the last layer's matrices: a layer's matrices are then one
        # contiguous range whose gradients are final as soon as the backward pass leaves the layer, while every
        # vector-shaped gradient (LayerNorm, biases: converted by one launch at the end of the pass) sits in the
        # tail of the buffer — which is what lets the gradient reduction start layer by layer under the backward pass
        ln_w = [(n, s) for n, s in decay if n.endswith("layer_norm.weight")]
        decay = [(n, s) for n, s in decay if not n.endswith("layer_norm.weight") and not n.startswith("__bottleneck__")] \
            + ln_w + [(n, s) for n, s in decay if n.startswith("__bottleneck__")]
        self.slots: dict[str, _Slot] = {}
        off = 0
        for n, s in decay:
            numel = math.prod(s)
            self.slots[n] = _Slot(off, s, numel)
            # q/k/v must stay adjacent (no padding between them): H*H and H are multiples of ALIGN
            off += (numel + ALIGN - 1) // ALIGN * ALIGN
        self.n_decay = off
        for n, s in nodecay:
            numel = math.prod(s)
            self.slots[n] = _Slot(off, s, numel)
            off += (numel + ALIGN - 1) // ALIGN * ALIGN
        self.numel = off
        if H % ALIGN != 0:
            raise ValueError(f"hidden size must be a multiple of {ALIGN}")
        dev = self.device
        self.p32 = guard.zeros(off, dtype=torch.float32, device=dev, name="encoder.p32")
        if act_dtype == torch.float32:
            self.p16 = self.p32
        elif p16_alloc is not None:
            self.p16 = p16_alloc(off, act_dtype)[:off]
        else:
            self.p16 = guard.zeros(off, dtype=act_dtype, device=dev, name="encoder.p16")
        if grad_alloc is not None and act_dtype != torch.float32:
            # the gradient buffer lives where the collective backend wants it (symmetric peer memory)
            self.g = grad_alloc(off, act_dtype)[:off]
        else:
            self.g = guard.zeros(off, dtype=act_dtype, device=dev, name="encoder.grad")
        self.m = guard.zeros(off, dtype=torch.float32, device=dev, name="encoder.adam_m")
        self.v = guard.zeros(off, dtype=torch.float32, device=dev, name="encoder.adam_v")
        self._init_params(seed)
        self._acts = None
        self._acts_key = None
        self._plan = None
        self.generation = 0
        self.own_gemm = False          # whether the current step's linears run on the own GEMM kernels
        self._own_mode = "0"
        self._own_supported = False
        self._wgrad_stream = None
        if self.device.type == "cuda" and act_dtype != torch.float32:
            from ..ops import cuda as cu
            # RENEE_B200_OWN_GEMM: 1 = the own tcgen05 GEMMs with fused epilogues always, 0 = library GEMMs + separate
            # element-wise kernels, auto (default) = own from OWN_GEMM_MIN_TOKENS tokens per step and GPU upwards
            self._own_mode = os.environ.get("RENEE_B200_OWN_GEMM", "auto")
            self._own_supported = cu.enc_gemm_supported(self.p16, H, Fd)
            self.own_gemm = self._own_supported and self._own_mode != "auto"
            if self._own_supported and os.environ.get("RENEE_B200_WGRAD_STREAM", "1") != "0":
                # weight-gradient GEMMs are off the critical path of the backward pass (nothing reads them before
                # the optimizer): they run on a second stream, where they fill the SMs that the data-gradient
                # GEMMs' last partial wave of tiles leaves idle (and, at small token counts, the SMs those GEMMs
                # never use).  Captured into the step's CUDA graph as parallel branches.
                self._wgrad_stream = torch.cuda.Stream(device=self.device)

    # ------------------------------------------------------------------ parameter views
    def view(self, buf: torch.Tensor, name: str) -> torch.Tensor:
        s = self.slots[name]
        return buf[s.offset: s.offset + s.numel].view(s.shape)

    def _qkv(self, buf, l, kind):
        p = f"transformer.layer.{l}.attention.q_lin.{kind}"
        s = self.slots[p]
        H = self.cfg.dim
        n = 3 * s.numel
        return buf[s.offset: s.offset + n].view((3 * H, H) if kind == "weight" else (3 * H,))

    def _init_params(self, seed: int) -> None:
        g = torch.Generator(device="cpu").manual_seed(int(seed))
        std = self.cfg.initializer_range
        for n, s in self.slots.items():
            if n.endswith("LayerNorm.weight") or n.endswith("layer_norm.weight"):
                t = torch.ones(s.shape)
            elif n.endswith("bias"):
                t = torch.zeros(s.shape)
            elif n.startswith("__bottleneck__"):
                stdv = 1.0 / math.sqrt(s.shape[1])
                t = (torch.rand(s.shape, generator=g) * 2 - 1) * stdv
            else:
                t = torch.randn(s.shape, generator=g) * std
                if n == "embeddings.word_embeddings.weight":
                    t[self.cfg.pad_token_id].zero_()
            self.view(self.p32, n).copy_(t)
        self.sync_compute_copy()

    def sync_compute_copy(self) -> None:
        if self.p16 is not self.p32:
            self.p16.copy_(self.p32)

    def encoder_state_dict(self) -> dict:
        return {n: self.view(self.p32, n).detach().clone() for n in self.encoder_param_names}

    def load_encoder_state_dict(self, sd: dict, strict: bool = True) -> None:
        missing = [n for n in self.encoder_param_names if n not in sd]
        if strict and missing:
            raise KeyError(f"missing encoder keys: {missing[:4]} ...")
        for n in self.encoder_param_names:
            if n in sd:
                self.view(self.p32, n).copy_(sd[n].to(self.p32.device, torch.float32))
        self.sync_compute_copy()

    def bottleneck_weight(self, buf=None):
        return self.view(self.p32 if buf is None else buf, "__bottleneck__.transformer_weight")

    # ------------------------------------------------------------------ activations
    def _alloc(self, b: int, S: int):
        key = (b, S)
        if self._acts_key is not None and self._acts_key[0] >= b and self._acts_key[1] == S:
            return
        cfg, dev, dt = self.cfg, self.device, self.act_dtype
        T, H, Fd, nh = b * S, cfg.dim, cfg.hidden_dim, cfg.n_heads
        e = lambda *shape, dtype=dt: guard.empty(*shape, dtype=dtype, device=dev, name=f"encoder.act{guard.registered()}")
        layers = []
        # long sequences: one softmax-gradient scratch serves every layer (it lives within one attention backward)
        att_ds = (e(b, nh, S, S) if S > 128 and dev.type == "cuda" and dt != torch.float32 else None)
        for _ in range(cfg.n_layers):
            layers.append(dict(qkv=e(T, 3 * H), ctx=e(T, H), ao=e(T, H), pre1=e(T, H), h1=e(T, H),
                               mean1=e(T, dtype=torch.float32), rstd1=e(T, dtype=torch.float32),
                               f1=e(T, Fd), a1=e(T, Fd), f2=e(T, H), pre2=e(T, H), h2=e(T, H),
                               mean2=e(T, dtype=torch.float32), rstd2=e(T, dtype=torch.float32),
                               att=ops.attention_workspace(b, S, nh, dev, dt, ds=att_ds)))
        self._acts = dict(h0=e(T, H), mean0=e(T, dtype=torch.float32), rstd0=e(T, dtype=torch.float32),
                          layers=layers, pooled=e(b, H, dtype=torch.float32),
                          dh=e(T, H), dh_b=e(T, H), dqkv=e(T, 3 * H), dctx=e(T, H), df1=e(T, Fd), da1=e(T, Fd),
                          emb=e(b, self.out_dims, dtype=torch.float32))
        self._acts_key = key
        self.generation += 1      # activation addresses changed: graphs captured over the old ones are stale

    # ------------------------------------------------------------------ forward
    def forward(self, input_ids: torch.Tensor, attention_mask: torch.Tensor, rng, train: bool = True) -> torch.Tensor:
        """ids/mask ``[b, S]`` int32 on the device → pooled embedding ``[b, D]`` fp32 (before the
        classifier-input dropout)."""
        cfg = self.cfg
        b, S = input_ids.shape
        self._alloc(b, S)
        A = self._acts
        T, H = b * S, cfg.dim
        if self._own_mode == "auto":
            self.own_gemm = self._own_supported and T >= OWN_GEMM_MIN_TOKENS
        P = self.p16
        pd = cfg.dropout if train else 0.0
        pa = cfg.attention_dropout if train else 0.0
        po = cfg.attn_output_dropout if train else 0.0
        self._fw = dict(ids=input_ids, mask=attention_mask, b=b, S=S, pd=pd, pa=pa, po=po, rng=rng)
        h = A["h0"][:T]
        ops.embed_ln_fwd(input_ids, self.view(P, "embeddings.word_embeddings.weight"),
                         self.view(P, "embeddings.position_embeddings.weight"),
                         self.view(P, "embeddings.LayerNorm.weight"), self.view(P, "embeddings.LayerNorm.bias"),
                         cfg.layer_norm_eps, S, pd, rng, _S_EMB, h, A["mean0"][:T], A["rstd0"][:T])
        if self.own_gemm:
            h = self._forward_layers_fused(h, attention_mask, T, pd, pa, po, rng)
        for l, L in enumerate(A["layers"] if not self.own_gemm else ()):
            pre = f"transformer.layer.{l}."
            sb = 8 * (l + 1)
            qkv = L["qkv"][:T]
            torch.mm(h, self._qkv(P, l, "weight").t(), out=qkv)
            ctx = L["ctx"][:T]
            ops.attention_fwd(qkv, self._qkv(P, l, "bias"), attention_mask, cfg.n_heads, pa, rng, sb + _S_PROBS,
                              ctx, L["att"])
            ao = L["ao"][:T]
            torch.mm(ctx, self.view(P, pre + "attention.out_lin.weight").t(), out=ao)
            h1 = L["h1"][:T]
            # HF DistilBERT applies no dropout to the attention output projection; BERT-family encoders do
            ops.bias_dropout_add_ln_fwd(ao, self.view(P, pre + "attention.out_lin.bias"), h,
                                        self.view(P, pre + "sa_layer_norm.weight"), self.view(P, pre + "sa_layer_norm.bias"),
                                        cfg.layer_norm_eps, po, rng, sb + _S_ATTN,
                                        h1, L["pre1"][:T], L["mean1"][:T], L["rstd1"][:T])
            f1 = L["f1"][:T]
            torch.mm(h1, self.view(P, pre + "ffn.lin1.weight").t(), out=f1)
            a1 = L["a1"][:T]
            ops.bias_gelu_fwd(f1, self.view(P, pre + "ffn.lin1.bias"), a1)
            f2 = L["f2"][:T]
            torch.mm(a1, self.view(P, pre + "ffn.lin2.weight").t(), out=f2)
            h2 = L["h2"][:T]
            ops.bias_dropout_add_ln_fwd(f2, self.view(P, pre + "ffn.lin2.bias"), h1,
                                        self.view(P, pre + "output_layer_norm.weight"),
                                        self.view(P, pre + "output_layer_norm.bias"),
                                        cfg.layer_norm_eps, pd, rng, sb + _S_FFN,
                                        h2, L["pre2"][:T], L["mean2"][:T], L["rstd2"][:T])
            L["h_in"] = h
            h = h2
        pooled = A["pooled"][:b]
        ops.pool_fwd(h.view(b, S, H), attention_mask, self.pooling, pooled)
        if self.bottleneck_dims > 0:
            emb = A["emb"][:b]
            torch.mm(pooled, self.bottleneck_weight().t(), out=emb)   # fp32, master weights
            return emb
        return pooled

    def _forward_layers_fused(self, h, attention_mask, T, pd, pa, po, rng):
        """The transformer blocks on the own GEMMs: 4 GEMMs, 1 attention and 2 LayerNorm launches per layer."""
        from ..ops import cuda as cu
        cfg, A, P = self.cfg, self._acts, self.p16
        for l, L in enumerate(A["layers"]):
            pre = f"transformer.layer.{l}."
            sb = 8 * (l + 1)
            qkv = L["qkv"][:T]
            cu.linear_fwd(h, self._qkv(P, l, "weight"), qkv)
            ctx = L["ctx"][:T]
            ops.attention_fwd(qkv, self._qkv(P, l, "bias"), attention_mask, cfg.n_heads, pa, rng, sb + _S_PROBS,
                              ctx, L["att"])
            pre1 = L["pre1"][:T]
            cu.linear_fwd(ctx, self.view(P, pre + "attention.out_lin.weight"), pre1, "bias_dropout_resid",
                          bias=self.view(P, pre + "attention.out_lin.bias"), resid=h, p=po, rng=rng, stream=sb + _S_ATTN)
            h1 = L["h1"][:T]
            cu.ln_fwd(pre1, self.view(P, pre + "sa_layer_norm.weight"), self.view(P, pre + "sa_layer_norm.bias"),
                      cfg.layer_norm_eps, h1, L["mean1"][:T], L["rstd1"][:T])
            a1 = L["a1"][:T]
            cu.linear_fwd(h1, self.view(P, pre + "ffn.lin1.weight"), a1, "bias_gelu",
                          bias=self.view(P, pre + "ffn.lin1.bias"), pre_out=L["f1"][:T])     # f1 holds x W^T + bias here
            pre2 = L["pre2"][:T]
            cu.linear_fwd(a1, self.view(P, pre + "ffn.lin2.weight"), pre2, "bias_dropout_resid",
                          bias=self.view(P, pre + "ffn.lin2.bias"), resid=h1, p=pd, rng=rng, stream=sb + _S_FFN)
            h2 = L["h2"][:T]
            cu.ln_fwd(pre2, self.view(P, pre + "output_layer_norm.weight"), self.view(P, pre + "output_layer_norm.bias"),
                      cfg.layer_norm_eps, h2, L["mean2"][:T], L["rstd2"][:T])
            L["h_in"] = h
            h = h2
        return h

    # ------------------------------------------------------------------ backward
    def backward(self, d_emb: torch.Tensor, on_layer_done=None) -> None:
        """``d_emb [b, D]`` fp32 → gradients of every parameter written into the flat ``g`` buffer
        (overwritten, not accumulated).  ``on_layer_done(l)`` is called when the gradients of layer ``l``'s
        matrices (one contiguous range of the flat buffer) have become final, and ``on_layer_done(-1)`` at the
        end of the pass (embeddings, bottleneck, LayerNorm parameters and biases), so a caller can reduce the
        buffer across ranks piece by piece while the remaining layers are still being differentiated."""
        if self.g.is_cuda:
            # column sums (LN gammas/betas, all bias gradients) are accumulated by the kernels and converted
            # by ONE launch at the end of the pass instead of a serial tail inside each kernel
            from ..ops import cuda as cu
            if self._plan is None:
                self._plan = cu.DeferredColumns(self.device, self.act_dtype)
            with cu.deferred_columns(self._plan):
                self._backward(d_emb, on_layer_done)
            self._plan.finalize()
        else:
            self._backward(d_emb, on_layer_done)
        if on_layer_done is not None:
            on_layer_done(-1)       # embeddings and every vector-shaped gradient are final: the whole buffer is

    def _wgrad(self, dy, x, dW) -> None:
        """``dW = dy^T x`` on the weight-gradient stream (ordered after everything issued so far on the current one)."""
        from ..ops import cuda as cu
        side = self._wgrad_stream
        if side is None:
            cu.linear_wgrad(dy, x, dW)
            return
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            cu.linear_wgrad(dy, x, dW)

    def _wgrad_join(self) -> None:
        """The current stream waits for the weight-gradient GEMMs issued so far (their inputs may be overwritten next)."""
        if self._wgrad_stream is not None:
            torch.cuda.current_stream().wait_stream(self._wgrad_stream)

    def _backward(self, d_emb: torch.Tensor, on_layer_done=None) -> None:
        cfg, A, fw = self.cfg, self._acts, self._fw
        b, S, pd, pa, rng = fw["b"], fw["S"], fw["pd"], fw["pa"], fw["rng"]
        T, H = b * S, cfg.dim
        P, G = self.p16, self.g
        mask = fw["mask"]
        if self.bottleneck_dims > 0:
            gw = self.view(G, "__bottleneck__.transformer_weight")
            pooled = A["pooled"][:b]
            if gw.dtype == torch.float32:
                torch.mm(d_emb.t(), pooled, out=gw)
            else:
                gw.copy_(torch.mm(d_emb.t(), pooled))
            d_pool = torch.mm(d_emb, self.bottleneck_weight())
        else:
            d_pool = d_emb
        dh = A["dh"][:T]
        ops.pool_bwd(d_pool, mask, self.pooling, S, dh.view(b, S, H))
        for l in reversed(range(cfg.n_layers)):
            L = A["layers"][l]
            pre = f"transformer.layer.{l}."
            sb = 8 * (l + 1)
            h_in = L["h_in"]
            # ---- output LN + FFN
            d_pre2, d_f2 = ops.bias_dropout_add_ln_bwd(
                dh, L["pre2"][:T], self.view(P, pre + "output_layer_norm.weight"), L["mean2"][:T], L["rstd2"][:T],
                pd, rng, sb + _S_FFN,
                self.view(G, pre + "output_layer_norm.weight"), self.view(G, pre + "output_layer_norm.bias"),
                self.view(G, pre + "ffn.lin2.bias"), A["dh_b"][:T], L["f2"][:T])
            if self.own_gemm:
                from ..ops import cuda as cu
                self._wgrad(d_f2, L["a1"][:T], self.view(G, pre + "ffn.lin2.weight"))
                df1 = A["df1"][:T]
                cu.linear_dgrad(d_f2, self.view(P, pre + "ffn.lin2.weight"), df1, "gelu_bwd", pre=L["f1"][:T],
                                dbias=self.view(G, pre + "ffn.lin1.bias"))
                self._wgrad(df1, L["h1"][:T], self.view(G, pre + "ffn.lin1.weight"))
                dh1 = cu.linear_dgrad(df1, self.view(P, pre + "ffn.lin1.weight"), dh, "add", resid=d_pre2)
                if d_f2 is d_pre2:
                    self._wgrad_join()      # without dropout d_f2 is the shared buffer the next kernel overwrites
                d_pre1, d_ao = ops.bias_dropout_add_ln_bwd(
                    dh1, L["pre1"][:T], self.view(P, pre + "sa_layer_norm.weight"), L["mean1"][:T], L["rstd1"][:T],
                    fw["po"], rng, sb + _S_ATTN,
                    self.view(G, pre + "sa_layer_norm.weight"), self.view(G, pre + "sa_layer_norm.bias"),
                    self.view(G, pre + "attention.out_lin.bias"), A["dh_b"][:T], L["ao"][:T])
                self._wgrad(d_ao, L["ctx"][:T], self.view(G, pre + "attention.out_lin.weight"))
                dctx = A["dctx"][:T]
                cu.linear_dgrad(d_ao, self.view(P, pre + "attention.out_lin.weight"), dctx)
                dqkv = A["dqkv"][:T]
                ops.attention_bwd(dctx, L["qkv"][:T], self._qkv(P, l, "bias"), mask, cfg.n_heads, pa, rng,
                                  sb + _S_PROBS, L["att"], dqkv, self._qkv(G, l, "bias"))
                self._wgrad(dqkv, h_in, self._qkv(G, l, "weight"))
                cu.linear_dgrad(dqkv, self._qkv(P, l, "weight"), dh, "add", resid=d_pre1)
                # the next layer overwrites the shared gradient buffers (dh_b, df1, dqkv) the GEMMs above read
                self._wgrad_join()
                if on_layer_done is not None:
                    on_layer_done(l)
                continue
            torch.mm(d_f2.t(), L["a1"][:T], out=self.view(G, pre + "ffn.lin2.weight"))
            da1 = A["da1"][:T]
            torch.mm(d_f2, self.view(P, pre + "ffn.lin2.weight"), out=da1)
            df1 = A["df1"][:T]
            ops.bias_gelu_bwd(da1, L["f1"][:T], self.view(P, pre + "ffn.lin1.bias"),
                              self.view(G, pre + "ffn.lin1.bias"), df1)
            torch.mm(df1.t(), L["h1"][:T], out=self.view(G, pre + "ffn.lin1.weight"))
            # dh1 = d_pre2 (residual) + df1 @ W1
            dh1 = torch.addmm(d_pre2, df1, self.view(P, pre + "ffn.lin1.weight"), out=dh)
            # ---- attention LN + attention
            d_pre1, d_ao = ops.bias_dropout_add_ln_bwd(
                dh1, L["pre1"][:T], self.view(P, pre + "sa_layer_norm.weight"), L["mean1"][:T], L["rstd1"][:T],
                fw["po"], rng, sb + _S_ATTN,
                self.view(G, pre + "sa_layer_norm.weight"), self.view(G, pre + "sa_layer_norm.bias"),
                self.view(G, pre + "attention.out_lin.bias"), A["dh_b"][:T], L["ao"][:T])
            torch.mm(d_ao.t(), L["ctx"][:T], out=self.view(G, pre + "attention.out_lin.weight"))
            dctx = A["dctx"][:T]
            torch.mm(d_ao, self.view(P, pre + "attention.out_lin.weight"), out=dctx)
            dqkv = A["dqkv"][:T]
            ops.attention_bwd(dctx, L["qkv"][:T], self._qkv(P, l, "bias"), mask, cfg.n_heads, pa, rng,
                              sb + _S_PROBS, L["att"], dqkv, self._qkv(G, l, "bias"))
            torch.mm(dqkv.t(), h_in, out=self._qkv(G, l, "weight"))
            torch.addmm(d_pre1, dqkv, self._qkv(P, l, "weight"), out=dh)
            if on_layer_done is not None:
                on_layer_done(l)
        ops.embed_ln_bwd(dh, fw["ids"], self.view(P, "embeddings.word_embeddings.weight"),
                         self.view(P, "embeddings.position_embeddings.weight"),
                         self.view(P, "embeddings.LayerNorm.weight"), A["mean0"][:T], A["rstd0"][:T],
                         S, pd, rng, _S_EMB, cfg.pad_token_id,
                         self.view(G, "embeddings.word_embeddings.weight"),
                         self.view(G, "embeddings.position_embeddings.weight"),
                         self.view(G, "embeddings.LayerNorm.weight"), self.view(G, "embeddings.LayerNorm.bias"))
