"""Exact top-K prediction over the label shards and the precision evaluator.

Parity: ``FullPredictor`` (reference dl_base.py:700-799) and ``PrecEvaluator`` (dl_base.py:801-861).

Prediction: every rank encodes its rows, embeddings are all-gathered, each rank takes the top-K of
its own label shard (on a GPU, K <= 8: a tcgen05 GEMM whose epilogue keeps a running top-8 per row, so the
``[B, Ls]`` logits are never written; larger K: per label chunk the logits GEMM followed by a row-wise selection
kernel; see ``ops/cuda.py::xfc_topk``), local label ids are offset to global ids and padded labels are
clipped to ``L-1``, candidates are merged across ranks, and rank 0 assembles a CSR score matrix
``[N_tst, L]`` with exactly K entries per row.

Evaluation: K=100 for the final epoch / ``--infer`` and 5 otherwise; rank 0 writes
``{name}_score_mat.npz``, filters reciprocal pairs, computes P/nDCG/PSP/PSnDCG@k, appends
``{name}_evaluation.tsv``; P@5 is broadcast and every rank saves its state dict on improvement.
"""
from __future__ import annotations

import datetime
import os

import numpy as np
import scipy.sparse as sp
import torch

from .utils.metrics import filter_predictions, metrics_table


class FullPredictor:
    def __init__(self, K: int = 5):
        self.K = K

    @torch.no_grad()
    def __call__(self, trainer, loader):
        n = len(loader.dataset)
        K = self.K
        L = trainer.sharding.num_labels
        Ls = trainer.sharding.labels_per_rank
        main = trainer.ctx.is_main
        if main:
            data = np.zeros((n, K), dtype=np.float32)
            inds = np.zeros((n, K), dtype=np.int32)
        ctr = 0
        D = None
        for batch in loader.epoch(0):
            B = batch.batch_size
            e = trainer.embed_eval(batch)
            if D is None:
                D = e.shape[1]
            X = torch.empty(B, D, dtype=e.dtype, device=e.device)
            X = trainer.comm.gather_embeddings(e, B, X)
            vals, idxs = trainer.local_topk(X, K)
            kk = vals.shape[1]
            if kk < K:  # shard smaller than K: pad with the lowest score so merges stay rectangular
                pad_v = torch.full((B, K - kk), torch.finfo(torch.float32).min, device=vals.device)
                pad_i = torch.zeros((B, K - kk), dtype=idxs.dtype, device=idxs.device)
                vals, idxs = torch.cat([vals.float(), pad_v], 1), torch.cat([idxs, pad_i], 1)
            idxs = idxs + trainer.rank * Ls
            idxs = idxs.clamp(max=L - 1)                      # padded labels → last real label
            vals, idxs = trainer.comm.merge_topk(vals.float().contiguous(), idxs.contiguous(), K)
            if main:
                data[ctr: ctr + B] = vals.float().cpu().numpy()
                inds[ctr: ctr + B] = idxs.cpu().numpy()
            ctr += B
        if not main:
            return None
        indptr = np.arange(0, n * K + 1, K)
        mat = sp.csr_matrix((data.ravel(), inds.ravel(), indptr), shape=(n, L))
        return mat


class PrecEvaluator:
    def __init__(self, loader, predictor: FullPredictor, true_labels: sp.spmatrix | None,
                 filter_mat: sp.spmatrix | None = None, K: int = 5, metric: str = "P", inv_prop=None,
                 final_k: int = 100):
        self.loader = loader
        self.predictor = predictor
        self.true_labels = true_labels
        self.filter_mat = filter_mat
        self.K = K
        self.metric = metric
        self.inv_prop = inv_prop
        self.final_k = final_k
        self.best_score = -9999999.0
        self.last_table = None

    def __call__(self, trainer, epoch: int = -1, loss: float = -1.0, out_dir: str | None = None, name: str = ""):
        main = trainer.ctx.is_main
        final = (epoch < 0) or (epoch == trainer.cfg.epochs - 1)
        self.predictor.K = self.final_k if final else 5
        score_mat = self.predictor(trainer, self.loader)
        score = 0.0
        prefix = f"{name}_" if name else ""
        if main:
            if out_dir:
                sp.save_npz(os.path.join(out_dir, f"{prefix}score_mat.npz"), score_mat)
            score_mat = filter_predictions(score_mat, self.filter_mat)
            res = metrics_table(score_mat, self.true_labels, self.inv_prop, K=max(5, self.K))
            self.last_table = res
            cols = ["epoch", "time", "loss", *[f"{m}@1" for m in res.index], *[f"{m}@3" for m in res.index],
                    *[f"{m}@{self.K}" for m in res.index]]
            row = [str(epoch), str(datetime.datetime.now()), "%.4E" % loss,
                   *["%.2f" % v for v in res["1"].values], *["%.2f" % v for v in res["3"].values],
                   *["%.2f" % v for v in res[str(self.K)].values]]
            if out_dir:
                out_file = os.path.join(out_dir, f"{prefix}evaluation.tsv")
                new = not os.path.exists(out_file)
                with open(out_file, "a") as f:
                    if new:
                        print("\t".join(cols), file=f)
                    print("\t".join(row), file=f)
            score = float(res[str(self.K)][self.metric])
        score = trainer.comm.broadcast_scalar(score, src=0)
        if score > self.best_score:
            if main:
                print(f"Rank {trainer.rank}: found best model with score : {'%.4f' % score}", flush=True)
                print("\t".join(cols))
                print("\t".join(row), flush=True)
            self.best_score = score
            trainer.best_score = score
            if out_dir:
                trainer.save(out_dir)
        return score
