"""Sharding invariance on CPU ranks (gloo): training with the label space split over 2 ranks gives
the same classifier and encoder as one rank, and prediction merges to the same top-K."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(rank, world, port, out_dir, default_impl):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from renee_b200.data import xcrepo
    from renee_b200.data.collate import GlobalBatchSampler, PrefetchLoader, XCCollator
    from renee_b200.data.synthetic import SyntheticSpec, SyntheticXC
    from renee_b200.evaluate import FullPredictor
    from renee_b200.models.encoder import EncoderConfig
    from renee_b200.parallel.dist import init_distributed, shutdown
    from renee_b200.train import TrainConfig, XCTrainer
    from renee_b200.utils.sharding import shard_labels

    torch.set_num_threads(2)
    ctx = init_distributed(rank, world, rank, device="cpu")
    enc = EncoderConfig(vocab_size=30522, max_position_embeddings=16, dim=128, n_layers=1, n_heads=2,
                        hidden_dim=256, dropout=0.0, attention_dropout=0.0)
    B = 12
    cfg = TrainConfig(batch_size=B // world, epochs=1, seed=0, dropout=0.0, lr1=0.05, lr2=1e-3, warmup=1,
                      wd1=1e-3, maxlen=16, fp32encoder=True, default_impl=default_impl)
    spec = SyntheticSpec(num_labels=320, seq_len=16, len_lo=4, len_hi=16, poisson_lam=2.0, seed=0)
    ids, mask, lab = SyntheticXC(spec).rows(np.arange(45))      # 45 rows: last batch is partial (9 rows)
    ds = xcrepo.InMemoryDataset(ids, mask, lab)
    sh = shard_labels(320, world)
    loader = PrefetchLoader(GlobalBatchSampler(45, B, True, 0), XCCollator(sh, ds, rank, 1, B, True, default_impl))
    tr = XCTrainer(cfg, enc, sh, ctx, steps_per_epoch=len(loader))
    if default_impl:   # give every world size the same global classifier
        g = torch.Generator().manual_seed(1)
        W = torch.randn(sh.padded_labels, 128, generator=g) * 0.02
        with torch.no_grad():
            tr.model.xfc_weight.copy_(W[rank * sh.labels_per_rank:(rank + 1) * sh.labels_per_rank])
    for batch in loader.epoch(0):
        tr.train_step(batch)
    tst = PrefetchLoader(GlobalBatchSampler(45, B, False, 0), XCCollator(sh, ds, rank, 1, B, False))
    score = FullPredictor(K=5)(tr, tst)
    sd = tr.state_dict()
    torch.save({"sd": sd, "score": score}, os.path.join(out_dir, f"w{world}_r{rank}_{int(default_impl)}.pt"))
    shutdown()


@pytest.mark.parametrize("default_impl", [False, True])
def test_two_ranks_equal_one_rank(tmp_path, default_impl):
    out = str(tmp_path)
    _run(0, 1, _free_port(), out, default_impl)
    mp.spawn(_run, args=(2, _free_port(), out, default_impl), nprocs=2, join=True)
    one = torch.load(os.path.join(out, f"w1_r0_{int(default_impl)}.pt"), weights_only=False)
    two = [torch.load(os.path.join(out, f"w2_r{r}_{int(default_impl)}.pt"), weights_only=False) for r in range(2)]
    W2 = torch.cat([t["sd"]["xfc_weight"] for t in two])
    torch.testing.assert_close(W2, one["sd"]["xfc_weight"], rtol=1e-3, atol=1e-5)
    for k, v in one["sd"].items():
        if k != "xfc_weight":
            # DDP semantics average encoder gradients over ranks (the reference does, main.py:161), so the
            # G=2 gradient is half the G=1 one; Adam removes the factor except where |g| ~ eps
            torch.testing.assert_close(two[0]["sd"][k], v, rtol=5e-2, atol=1e-3, msg=lambda m: f"{k}: {m}")
            torch.testing.assert_close(two[1]["sd"][k], two[0]["sd"][k], rtol=0, atol=0)
    a, b = one["score"], two[0]["score"]
    assert two[1]["score"] is None and a.shape == b.shape == (45, 320)
    assert (abs(a - b) > 1e-4).nnz == 0
