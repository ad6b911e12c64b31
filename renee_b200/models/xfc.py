"""Label-sharded extreme classifier: state and the loss-skipping training step.

Parity targets in the reference: ``xfc_weight [Ls, D]`` initialised N(0, 0.02) (dl_base.py:185-187);
the manual forward/backward ``BCELossMultiNode.xfc_forward/xfc_backward`` (dl_base.py:568-642);
apex FusedSGD for the update (main.py:177-179, dl_base.py:343-344); split gradient accumulation
(dl_base.py:317-340).

Per step and per rank, with ``X [B, D]`` the gathered embeddings of the global batch::

    Gt = sigmoid(W Xᵀ) − Yᵀ            [Ls, B]   (never the loss, never dense Y)
    dX = scale · Gtᵀ W                  [B, D]    fp32, summed over ranks by the caller
    dW = Gt X ; g = dW + wd·W ; M = mo·M + g ; W −= lr·M

Differences from the reference, made for B200:

* ``--fp16xfc`` stores ``W`` and the momentum ``M`` in fp16 (the reference keeps fp32 masters and
  casts every step, dl_base.py:562); the update is computed in fp32 inside the dW kernel's epilogue
  and written back once.  The new weights are rounded STOCHASTICALLY by default: with round-to-nearest
  an update ``lr·M`` below half an fp16 ulp of ``W`` (about 1.5e-5 at ``|W|`` = 0.03) is dropped on every
  step, which late in the cosine schedule silently freezes tail labels; stochastic rounding keeps the
  expected update exact (``tests/test_xfc_step.py`` bounds both against fp32 masters over several hundred
  small steps).  ``stochastic_round=False`` / ``--no-stochastic-round`` restores round-to-nearest;
* split accumulation chunks the **label** dimension rather than the batch rows: a chunk's ``dW`` is
  then complete, so the SGD update stays fused and no ``[Ls, D]`` fp32 gradient buffer exists, while
  the scratch ``Gt`` is bounded to ``B · Ls/accum`` elements exactly as ``--accum`` intends.  Chunks
  are additionally capped so that ``Gt`` stays L2-resident between the three kernels;
* positives arrive sorted by label, so a chunk (and inside the kernel a 128-label tile) finds its
  entries by binary search.
"""
from __future__ import annotations

import os

import torch

from ..ops import reference as ref
from ..utils import guard

INIT_CHUNK = 1 << 16
GT_L2_BUDGET_BYTES = 128 << 20  # bound of the Gt scratch; measured: larger chunks amortise the kernels' fill and drain
                                # better than an L2-resident Gt pays (3.98 -> 3.92 ms at 131 K labels, 48 -> 96 MB)


class XFCClassifier:
    def __init__(self, labels_per_rank: int, dims: int, device, fp16: bool, rank: int = 0,
                 seed: int = 42, init_std: float = 0.02, max_batch: int = 1024, accum: int = 1,
                 stochastic_round: bool = True):
        self.Ls = int(labels_per_rank)
        self.D = int(dims)
        self.device = torch.device(device)
        self.dtype = torch.float16 if fp16 else torch.float32
        self.rank = rank
        self.accum = max(1, int(accum))
        self.max_batch = int(max_batch)
        self.stochastic_round = bool(stochastic_round)
        self.W = guard.empty(self.Ls, self.D, dtype=self.dtype, device=self.device, name="xfc.W")
        self.M = guard.zeros(self.Ls, self.D, dtype=self.dtype, device=self.device, name="xfc.M")
        self._init_weight(seed, init_std)
        self.chunk = self._pick_chunk()
        self._scratch = None

    # ------------------------------------------------------------------ init / io
    def _init_weight(self, seed: int, std: float) -> None:
        """Rows are generated in fixed chunks keyed by their GLOBAL label index, so the assembled
        ``[Lp, D]`` matrix does not depend on the number of ranks (the reference seeds every rank
        identically, which makes all shards start equal — main.py:22, dl_base.py:187)."""
        if self.device.type == "meta":      # size-accounting dry runs (utils/memory_plan.py): nothing to fill
            return
        lo = self.rank * self.Ls
        hi = lo + self.Ls
        g = torch.Generator(device=self.device)
        c0 = lo // INIT_CHUNK
        c1 = (hi + INIT_CHUNK - 1) // INIT_CHUNK
        for c in range(c0, c1):
            g.manual_seed(int(seed) * 1000003 + c)
            block = torch.randn(INIT_CHUNK, self.D, generator=g, device=self.device, dtype=torch.float32) * std
            a = max(lo, c * INIT_CHUNK)
            b = min(hi, (c + 1) * INIT_CHUNK)
            self.W[a - lo: b - lo].copy_(block[a - c * INIT_CHUNK: b - c * INIT_CHUNK])

    def _pick_chunk(self) -> int:
        per_accum = (self.Ls + self.accum - 1) // self.accum
        budget = int(float(os.environ.get("RENEE_B200_XFC_GT_MB", GT_L2_BUDGET_BYTES / (1 << 20))) * (1 << 20))
        cap = max(128, budget // (2 * max(self.max_batch, 1)))
        chunk = min(per_accum, cap)
        return max(128, (chunk + 127) // 128 * 128)

    def state_dict_weight(self) -> torch.Tensor:
        return self.W.detach().float().clone()

    def load_weight(self, w: torch.Tensor) -> None:
        self.W.copy_(w.to(self.device, self.dtype))

    def optimizer_state_dict(self) -> dict:
        return {"momentum_buffer": self.M.detach().clone()}

    def load_optimizer_state_dict(self, sd: dict) -> None:
        self.M.copy_(sd["momentum_buffer"].to(self.device, self.dtype))

    # ------------------------------------------------------------------ training step
    def scratch(self, B: int):
        if self._scratch is None or self._scratch["B"] < B:
            chunk = min(self.chunk, (self.Ls + 127) // 128 * 128)
            ldg = (B + 7) // 8 * 8
            self._scratch = {"B": B, "Gt": guard.empty(chunk * ldg, dtype=torch.float16 if self.dtype == torch.float16 else torch.float32,
                                                      device=self.device, name="xfc.Gt")}
        return self._scratch

    def step(self, X: torch.Tensor, pos_rows: torch.Tensor, pos_labels: torch.Tensor, nnz,
             dX_out: torch.Tensor, hp, mo: float, wd: float, want_loss: bool = False, wait=None, signal=None,
             side_stream=None):
        """One classifier step on this rank's shard.

        ``X [B, D]`` in the classifier dtype; ``pos_rows/pos_labels`` int32 sorted by label (only the
        first ``nnz`` entries are valid; ``nnz`` may be a device tensor on the kernel path);
        ``dX_out [B, D]`` fp32 receives ``scale · Gᵀ W`` (overwritten).  The learning rate and loss
        scale are read from ``hp``.  Returns the sparse BCE loss sum (fp32 tensor) or ``None``."""
        if X.is_cuda and self.dtype == torch.float16:
            from ..ops import cuda as cu
            return cu.xfc_step(self, X, pos_rows, pos_labels, nnz, dX_out, hp, mo, wd, want_loss, wait, signal, side_stream)
        if wait is not None or signal is not None:
            raise RuntimeError("the fused collectives need the fp16 classifier kernels (--fp16xfc on a GPU)")
        return self._step_reference(X, pos_rows, pos_labels, nnz, dX_out, hp, mo, wd, want_loss)

    def _step_reference(self, X, pos_rows, pos_labels, nnz, dX_out, hp, mo, wd, want_loss):
        from ..optim.hparams import HP
        n = int(nnz)
        rows, labels = pos_rows[:n].long(), pos_labels[:n].long()
        lr = float(hp.buf[HP.LR_XFC])
        scale = float(hp.buf[HP.SCALE])
        dX_out.zero_()
        loss = torch.zeros((), dtype=torch.float32, device=X.device) if want_loss else None
        for l0 in range(0, self.Ls, self.chunk):
            l1 = min(self.Ls, l0 + self.chunk)
            sel = (labels >= l0) & (labels < l1)
            Gt, l = ref.xfc_logit_grad(X, self.W[l0:l1], rows[sel], labels[sel] - l0, want_loss)
            if want_loss:
                loss += l
            dX_out += ref.xfc_dx(Gt, self.W[l0:l1], scale)
            ref.xfc_dw_sgd(Gt, X, self.W[l0:l1], self.M[l0:l1], lr, mo, wd)
        return loss

    # ------------------------------------------------------------------ inference
    def topk(self, X: torch.Tensor, k: int):
        """Local top-k over this shard: ``(values [B,k] fp32, local label ids [B,k] int64)``."""
        if X.is_cuda and self.dtype == torch.float16:
            from ..ops import cuda as cu
            return cu.xfc_topk(self, X, k)
        vals, idxs = None, None
        for l0 in range(0, self.Ls, self.chunk):
            l1 = min(self.Ls, l0 + self.chunk)
            v, i = ref.topk_logits(X, self.W[l0:l1], k)
            i = i + l0
            if vals is None:
                vals, idxs = v, i
            else:
                cv, ci = torch.cat([vals, v], 1), torch.cat([idxs, i], 1)
                vals, sel = torch.topk(cv, min(k, cv.shape[1]), dim=1)
                idxs = torch.gather(ci, 1, sel)
        return vals, idxs
