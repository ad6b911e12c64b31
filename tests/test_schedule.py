"""Cosine-with-warmup multiplier equals transformers' scheduler (reference dl_base.py:395-397)."""
import torch

from renee_b200.optim.schedule import CosineWarmupSchedule, cosine_warmup_multiplier


def test_matches_transformers():
    import transformers
    p = torch.nn.Parameter(torch.zeros(1))
    opt = torch.optim.SGD([p], lr=0.05)
    sched = transformers.get_cosine_schedule_with_warmup(opt, num_warmup_steps=7, num_training_steps=50)
    mine = CosineWarmupSchedule(0.05, 7, 50)
    for step in range(50):
        assert abs(opt.param_groups[0]["lr"] - mine.lr()) < 1e-12, step
        opt.step(); sched.step(); mine.step()


def test_state_roundtrip():
    a = CosineWarmupSchedule(1.0, 3, 20)
    for _ in range(5):
        a.step()
    b = CosineWarmupSchedule(0.0, 0, 1)
    b.load_state_dict(a.state_dict())
    assert b.lr() == a.lr() and cosine_warmup_multiplier(5, 3, 20) == a.multiplier()
