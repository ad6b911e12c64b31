"""Optimized (manual, loss-skipping) training equals the autograd default path step for step."""
import numpy as np
import pytest
import torch

from renee_b200.data import xcrepo
from renee_b200.data.collate import GlobalBatchSampler, PrefetchLoader, XCCollator
from renee_b200.data.synthetic import SyntheticSpec, SyntheticXC
from renee_b200.models.encoder import EncoderConfig
from renee_b200.parallel.dist import DistContext
from renee_b200.train import TrainConfig, XCTrainer, normalise_state_dict_keys
from renee_b200.utils.sharding import shard_labels


def make(default_impl, tmp=None, **kw):
    enc = EncoderConfig(vocab_size=30522, max_position_embeddings=32, dim=128, n_layers=2, n_heads=2,
                        hidden_dim=512, dropout=0.0, attention_dropout=0.0)
    base = dict(batch_size=16, epochs=2, seed=0, dropout=0.0, lr1=0.05, lr2=1e-3, warmup=2, wd1=1e-3, wd2=0.01,
                default_impl=default_impl, maxlen=16, fp32encoder=True, out_dir=str(tmp) if tmp else "")
    base.update(kw)
    cfg = TrainConfig(**base)
    spec = SyntheticSpec(num_labels=512, seq_len=16, len_lo=4, len_hi=16, poisson_lam=2.0, seed=0)
    ids, mask, lab = SyntheticXC(spec).rows(np.arange(64))
    ds = xcrepo.InMemoryDataset(ids, mask, lab)
    sh = shard_labels(512, 1)
    loader = PrefetchLoader(GlobalBatchSampler(64, 16, True, 0), XCCollator(sh, ds, 0, 1, 16, True, default_impl))
    tr = XCTrainer(cfg, enc, sh, DistContext(), steps_per_epoch=len(loader))
    return tr, loader


def test_optimized_equals_default_for_several_steps():
    a, la = make(False)
    b, lb = make(True)
    a.load_state_dict(b.state_dict())
    losses = []
    for batch_a, batch_b in zip(la.epoch(0), lb.epoch(0)):
        a.train_step(batch_a)
        b.train_step(batch_b)
        losses.append((a.pop_loss(), b.pop_loss()))
    sa, sb = a.state_dict(), b.state_dict()
    assert set(sa) == set(sb)
    for k in sa:
        torch.testing.assert_close(sa[k], sb[k], rtol=2e-3, atol=2e-5, msg=lambda m: f"{k}: {m}")
    la_, lb_ = losses[0]
    assert abs(la_ - lb_) < 1e-5       # first step is a sampling step (count % 100 == 0)


def test_state_dict_layout_and_prefix_variants(tmp_path):
    tr, _ = make(False, tmp_path, bottleneck_dims=64)
    sd = tr.state_dict()
    assert sd["xfc_weight"].shape == (512, 64) and sd["xfc_weight"].dtype == torch.float32
    assert "embed.0.transformer.embeddings.word_embeddings.weight" in sd
    assert "embed.0.transformer.transformer.layer.1.ffn.lin2.bias" in sd
    assert sd["embed.1.transformer_weight"].shape == (64, 128)
    wrapped = {k.replace("embed.", "embed.module.", 1).replace("embed.module.0.", "embed.module.0._orig_mod."): v
               for k, v in sd.items()}
    assert set(normalise_state_dict_keys(wrapped)) == set(sd)
    tr2, _ = make(False, tmp_path, bottleneck_dims=64, seed=5)
    tr2.load_state_dict(wrapped)
    for k, v in tr2.state_dict().items():
        torch.testing.assert_close(v, sd[k])
    path = tr.save()
    assert path.endswith("renee-exp_0_state_dict.pt")
    tr2.load()


def test_checkpoint_resume_is_bitwise_deterministic(tmp_path):
    ck = str(tmp_path / "ck")
    full, lf = make(False, dropout=0.3, checkpoint_resume="", epochs=2)
    full.fit(lf, log=lambda *a: None)
    first, l1 = make(False, dropout=0.3, checkpoint_resume=ck, epochs=1)
    first.total_steps = full.total_steps
    first.xfc_sched.total_steps = first.tf_sched.total_steps = full.total_steps
    first.fit(l1, log=lambda *a: None)
    second, l2 = make(False, dropout=0.3, checkpoint_resume=ck, epochs=2)
    second.fit(l2, log=lambda *a: None)
    assert second.count == full.count
    for k, v in full.state_dict().items():
        assert torch.equal(v, second.state_dict()[k]), k
    import os
    assert os.path.exists(os.path.join(ck, "renee-exp_0_checkpoint.pt"))
    assert os.path.exists(os.path.join(ck, "renee-exp_0_checkpoint_prev.pt"))


def test_loss_scale_state_machine_skips_and_backs_off():
    from renee_b200.optim.hparams import HP, HyperParams
    hp = HyperParams("cpu", init_scale=2.0 ** 12, growth_interval=3)
    hp.buf[HP.FOUND_INF] = 1.0
    hp.update_scale()
    assert hp.get_scale() == 2.0 ** 11 and float(hp.buf[HP.ADAM_STEP]) == 0 and float(hp.buf[HP.FOUND_INF]) == 0
    for _ in range(3):
        hp.update_scale()
    assert hp.get_scale() == 2.0 ** 12 and float(hp.buf[HP.ADAM_STEP]) == 3
    off = HyperParams("cpu", enabled=False)
    assert off.get_scale() == 1.0


def _fit_with_accum(accum, tmp_path, device="cpu", n=40, **kw):
    """Trainer + loaders built the way ``cli.start`` builds them (global batch 16, 40 rows: the last batch of an
    epoch is partial), one epoch."""
    enc = EncoderConfig(vocab_size=30522, max_position_embeddings=32, dim=128, n_layers=2, n_heads=2,
                        hidden_dim=512, dropout=0.0, attention_dropout=0.0)
    base = dict(batch_size=16, epochs=1, seed=0, dropout=0.0, lr1=0.05, lr2=1e-3, warmup=2, wd1=1e-3, wd2=0.01,
                maxlen=16, fp32encoder=True, accum=accum, noloss=True)
    base.update(kw)
    cfg = TrainConfig(**base)
    spec = SyntheticSpec(num_labels=700, seq_len=16, len_lo=4, len_hi=16, poisson_lam=2.0, seed=0)
    ids, mask, lab = SyntheticXC(spec).rows(np.arange(n))
    ds = xcrepo.InMemoryDataset(ids, mask, lab)
    sh = shard_labels(700, 1)
    gbsz = cfg.batch_size
    loader = PrefetchLoader(GlobalBatchSampler(n, gbsz, True, 0),
                            XCCollator(sh, ds, 0, accum, max(1, gbsz // accum), True, False))
    tr = XCTrainer(cfg, enc, sh, DistContext(device=torch.device(device)), steps_per_epoch=len(loader))
    tr.fit(loader, log=lambda *a: None)
    return tr


def test_accum_through_the_loader_equals_accum_one(tmp_path):
    """``--accum`` only bounds the classifier scratch (dl_base.py:317-340): the trained weights must not depend on it."""
    ref = _fit_with_accum(1, tmp_path)
    sd = ref.state_dict()
    for accum in (2, 4):
        tr = _fit_with_accum(accum, tmp_path)
        assert tr.xfc.chunk <= (tr.Ls + accum - 1) // accum + 127      # Gt scratch is B x Ls/accum (128-label granularity)
        for k, v in tr.state_dict().items():
            if "k_lin.bias" in k:
                continue        # its true gradient is zero (softmax is shift-invariant): Adam amplifies rounding noise
            torch.testing.assert_close(v, sd[k], rtol=1e-3, atol=1e-5, msg=lambda m: f"accum={accum} {k}: {m}")


def test_flat_moments_are_remapped_by_name_when_the_layout_differs():
    """The flat AdamW moments of a checkpoint written under another ordering of the flat buffer land at the right
    parameters (and a parameter of another size is refused)."""
    from types import SimpleNamespace
    from renee_b200 import checkpoint as ck

    def slot(o, k):
        return SimpleNamespace(offset=o, numel=k)
    enc = SimpleNamespace(slots={"b": slot(0, 4), "a": slot(4, 2)}, m=torch.zeros(6), v=torch.zeros(6))
    old = {"layout": [("a", 0, 2), ("b", 2, 4)], "exp_avg": torch.arange(6.), "exp_avg_sq": torch.arange(6.) * 10}
    ck._load_flat_moments(enc, old, "cpu")
    assert enc.m.tolist() == [2., 3., 4., 5., 0., 1.]
    assert enc.v.tolist() == [20., 30., 40., 50., 0., 10.]
    same = {"layout": ck._flat_layout(enc), "exp_avg": torch.ones(6), "exp_avg_sq": torch.ones(6)}
    ck._load_flat_moments(enc, same, "cpu")
    assert enc.m.tolist() == [1.] * 6
    bad = {"layout": [("a", 0, 3), ("b", 3, 3)], "exp_avg": torch.ones(6), "exp_avg_sq": torch.ones(6)}
    with pytest.raises(RuntimeError):
        ck._load_flat_moments(enc, bad, "cpu")
