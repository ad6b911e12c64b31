"""Collectives of the hybrid data/model-parallel step.

Three exchanges happen every training step (reference call sites in parentheses):

* all-gather of each rank's ``[b, D]`` embeddings into the global ``X [B, D]`` (dl_base.py:535-558);
* summation of the per-rank partial ``dX [B, D]`` — the reference all-reduces the full matrix
  (dl_base.py:617) although a rank only consumes its own rows; this package reduce-scatters;
* averaging of the encoder gradients (DDP, main.py:161).

plus the small ones: sampled-loss scalar (dl_base.py:587), top-K merge (dl_base.py:774-779) and the
P@5 broadcast (dl_base.py:848).

:class:`TorchCollectives` is the library baseline (NCCL on GPUs, gloo on CPU) and the semantic
reference; :class:`renee_b200.parallel.fused.PeerCollectives` replaces the data path with
hand-written kernels over NVLink peer memory.  Both handle a partial final batch whose rows are not
evenly divisible: rank ``r`` owns rows ``batch_row_range(B, G, r)``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..utils.sharding import batch_row_range
from .dist import DistContext


class TorchCollectives:
    def __init__(self, ctx: DistContext):
        self.ctx = ctx
        self.G = ctx.world_size
        self.rank = ctx.rank

    # ---- step protocol used by the trainer (the fused backend overrides these)
    @property
    def graph_safe(self) -> bool:
        """Whether the step may be replayed from a CUDA graph: yes on one rank (no collectives at all);
        the library collectives of several ranks are launched eagerly."""
        return self.G == 1

    def setup(self, B_max: int, D: int) -> None:
        pass

    def host_begin(self) -> None:
        pass

    def device_begin(self) -> None:
        pass

    @property
    def parity(self) -> int:
        return 0

    def embeddings_to_X(self, emb, B, p, rng, stream_id, bufs):
        """Classifier-input dropout + cast of this rank's pooled embeddings, then the all-gather.
        Returns ``(X [B, D], wait)``; ``wait`` is what the logits GEMM must wait for (``None`` here:
        the library collective has completed in stream order)."""
        from .. import ops
        b = emb.shape[0]
        x_local = bufs["x_local"][:b]
        ops.dropout_cast_fwd(emb, p, rng, stream_id, x_local)
        return self.gather_embeddings(x_local, B, bufs["X"]), None

    def dx_buffer(self, B, bufs):
        """Buffer the dX GEMM accumulates into, and the signal its last CTA has to raise (none)."""
        return bufs["dX"][:B], None

    def dx_to_local(self, dX, B, p, rng, stream_id, bufs):
        """Sum of dX over ranks restricted to this rank's rows, with the dropout backward applied."""
        from .. import ops
        dx_local = self.reduce_scatter_dx(dX, B, bufs["dx_local"])
        de = bufs["de"][: dx_local.shape[0]]
        ops.dropout_bwd(dx_local, p, rng, stream_id, de)
        return de

    def optimizer_step(self, enc, hp, beta1, beta2, eps, wd) -> None:
        """Reduce the encoder gradients over ranks and apply AdamW (here: all-reduce, then the full fused
        AdamW on every rank).  The fused backend shards this step across ranks."""
        from .. import ops
        grad_mult = self.allreduce_grads(enc.g, hp)
        ops.adamw_step(enc.p32, enc.m, enc.v, enc.g, enc.p16, hp, beta1, beta2, eps, wd, enc.n_decay, grad_mult)

    def sync_master(self, enc) -> None:
        """Make every rank's fp32 master weights complete (a no-op unless the optimizer is sharded)."""

    # ---- embeddings
    def gather_embeddings(self, x_local: torch.Tensor, B: int, out: torch.Tensor) -> torch.Tensor:
        """``x_local [b_r, D]`` → ``out[:B]`` with rank r's rows at ``batch_row_range(B, G, r)``."""
        if self.G == 1:
            out[:B].copy_(x_local)
            return out[:B]
        per = (B + self.G - 1) // self.G
        D = x_local.shape[1]
        pad = torch.zeros(per, D, dtype=x_local.dtype, device=x_local.device)
        pad[: x_local.shape[0]].copy_(x_local)
        parts = [torch.empty_like(pad) for _ in range(self.G)]
        dist.all_gather(parts, pad)
        for r in range(self.G):
            s, e = batch_row_range(B, self.G, r)
            out[s:e].copy_(parts[r][: e - s])
        return out[:B]

    # ---- dX
    def reduce_scatter_dx(self, dX: torch.Tensor, B: int, out: torch.Tensor) -> torch.Tensor:
        """Sum ``dX [B, D]`` over ranks; rank r receives its own rows in ``out[:b_r]``."""
        s, e = batch_row_range(B, self.G, self.rank)
        if self.G == 1:
            out[: e - s].copy_(dX[s:e])
            return out[: e - s]
        if B % self.G == 0 and dX.is_cuda:
            dist.reduce_scatter_tensor(out[: e - s], dX[:B].contiguous())
        else:
            buf = dX[:B].contiguous()
            dist.all_reduce(buf)
            out[: e - s].copy_(buf[s:e])
        return out[: e - s]

    # ---- encoder gradients
    def allreduce_grads(self, g: torch.Tensor, hp) -> float:
        """Sum the flat gradient buffer over ranks and raise ``hp``'s found-inf flag if any element is
        non-finite.  Returns the factor the optimizer still has to apply to obtain the MEAN over ranks
        (DDP semantics, reference main.py:161) — folded into the fused AdamW's unscale multiply."""
        from ..optim.hparams import HP
        if self.G > 1:
            dist.all_reduce(g)
        if g.is_cuda:
            from ..ops import cuda as cu
            cu.grad_check(g, hp)
        else:
            bad = (~torch.isfinite(g)).any().to(torch.float32)
            hp.buf[HP.FOUND_INF] = torch.maximum(hp.buf[HP.FOUND_INF], bad)
        return 1.0 / self.G

    # ---- small exchanges
    def allreduce_scalar(self, t: torch.Tensor) -> torch.Tensor:
        if self.G > 1:
            dist.all_reduce(t)
        return t

    def broadcast_scalar(self, value: float, src: int = 0) -> float:
        if self.G == 1:
            return value
        t = torch.tensor([value], dtype=torch.float32, device=self.ctx.device)
        dist.broadcast(t, src=src)
        return float(t.item())

    def merge_topk(self, vals: torch.Tensor, idxs: torch.Tensor, k: int):
        """``vals/idxs [n, k]`` per rank (global label ids) → global top-k on every rank."""
        if self.G == 1:
            return vals, idxs
        v_parts = [torch.empty_like(vals) for _ in range(self.G)]
        i_parts = [torch.empty_like(idxs) for _ in range(self.G)]
        dist.all_gather(v_parts, vals.contiguous())
        dist.all_gather(i_parts, idxs.contiguous())
        cv, ci = torch.cat(v_parts, 1), torch.cat(i_parts, 1)
        v, sel = torch.topk(cv, min(k, cv.shape[1]), dim=1)
        return v, torch.gather(ci, 1, sel)

    def barrier(self) -> None:
        self.ctx.barrier()
