"""Peer-memory collective kernels on ONE GPU with emulated ranks.

Every kernel either signals or waits for a given flag class, so the emulated ranks' kernels can be run
one after another on a single device (all signals of a phase first, then the waiters): nothing ever
waits for a kernel that has not run yet.  Each emulated rank has its own buffers; the "peer pointer"
tables simply point at the other rank's buffers on the same GPU.  The last test lets a bounded wait
run out on a flag that nothing sets and checks that the kernel returns with a status code and that
the context stays usable.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

from renee_b200 import ops
from renee_b200.ops import reference as ref
from renee_b200.optim.hparams import HP, HyperParams
from renee_b200.parallel.fused import F_AG, F_ARA, F_ARB, F_FOUND, F_RS, FLAG_WORDS
from renee_b200.utils.sharding import batch_row_range


def dev():
    return torch.device("cuda", 0)


def cu():
    from renee_b200.ops import cuda
    return cuda


class Rank:
    def __init__(self, r, G, rows, D, n_grad):
        self.r = r
        self.flags = torch.zeros(FLAG_WORDS, dtype=torch.int32, device=dev())
        self.X = torch.zeros(rows, D, dtype=torch.float16, device=dev())
        self.dXp = torch.zeros(rows, D, dtype=torch.float32, device=dev())
        self.grad = torch.zeros(n_grad, dtype=torch.bfloat16, device=dev())
        self.step = torch.ones(1, dtype=torch.int32, device=dev())
        self.counters = torch.zeros(64, dtype=torch.int32, device=dev())
        self.seed = torch.tensor([77 + r], dtype=torch.int32, device=dev())
        self.rng = ops.StepRNG(77 + r, self.seed)


@pytest.mark.parametrize("G,B", [(2, 64), (4, 250)])
def test_allgather_logits_dx_reducescatter_emulated(G, B):
    torch.manual_seed(0)
    D, Ls, p = 128, 640, 0.3
    ranks = [Rank(r, G, B + G, D, 1024) for r in range(G)]
    x_ptrs = cu().ptr_array([k.X.data_ptr() for k in ranks])
    f_ptrs = cu().ptr_array([k.flags.data_ptr() for k in ranks])
    d_ptrs = cu().ptr_array([k.dXp.data_ptr() for k in ranks])
    embs, want_rows = [], []
    for k in ranks:
        s, e = batch_row_range(B, G, k.r)
        emb = torch.randn(e - s, D, device=dev())
        embs.append(emb)
        want_rows.append(ref.dropout_cast_fwd(emb, p, k.rng.seed, 5, torch.float16))
        cu().ag_push(emb, p, k.rng, 5, x_ptrs, s, f_ptrs, F_AG, k.r, G, k.step, k.counters)
    X_want = torch.cat(want_rows)
    for k in ranks:
        torch.testing.assert_close(k.X[:B], X_want, rtol=0, atol=0)
        assert k.flags[F_AG:F_AG + G].tolist() == [1] * G
    # every rank owns a label shard; the logits GEMM waits on the all-gather flags (already raised)
    Ws = [(torch.randn(Ls, D, device=dev()) * 0.05).half() for _ in ranks]
    hp = HyperParams(dev(), init_scale=8.0)
    ldG = (B + 7) // 8 * 8
    n0 = torch.zeros(1, dtype=torch.int32, device=dev())
    empty = torch.zeros(1, dtype=torch.int32, device=dev())
    partial_want = []
    for k, W in zip(ranks, Ws):
        Gt = torch.zeros(Ls, ldG, dtype=torch.float16, device=dev())
        cu().xfc_logits_grad(W, k.X[:B], Gt, ldG, empty, empty, n0, 0, wait=(k.flags[F_AG:], G, k.step))
        Gr, _ = ref.xfc_logit_grad(X_want, W, empty[:0], empty[:0])
        torch.testing.assert_close(Gt[:, :B].float(), Gr.float(), rtol=2e-3, atol=2e-3)
        cu().xfc_dx(Gt, ldG, W, B, k.dXp[:B], hp.buf, 3, signal=(k.counters[32:], f_ptrs, G, F_RS + k.r, k.step))
        partial_want.append(ref.xfc_dx(Gr, W, 8.0))
    cu().check_status()
    total = sum(partial_want)
    for k in ranks:
        assert k.flags[F_RS:F_RS + G].tolist() == [1] * G
        s, e = batch_row_range(B, G, k.r)
        de = torch.empty(e - s, D, device=dev())
        cu().rs_pull(d_ptrs, G, s, e - s, D, de, k.flags[F_RS:], k.step, p, k.rng, 5)
        want = ref.dropout_bwd(total[s:e], p, k.rng.seed, 5)
        torch.testing.assert_close(de, want, rtol=2e-3, atol=8.0 * 2e-3)
    cu().check_status()


def test_grad_allreduce_emulated_and_found_inf():
    G, n = 4, 8 * 1000 + 8 * 3
    torch.manual_seed(1)
    ranks = [Rank(r, G, 8, 8, n) for r in range(G)]
    for k in ranks:
        k.grad.copy_((torch.randn(n, device=dev()) * 3).bfloat16())
    want = sum(k.grad.float() for k in ranks)
    g_ptrs = cu().ptr_array([k.grad.data_ptr() for k in ranks])
    f_ptrs = cu().ptr_array([k.flags.data_ptr() for k in ranks])
    hps = [HyperParams(dev()) for _ in ranks]
    for rnd in range(2):
        if rnd == 1:
            for k in ranks:
                k.step += 1
                k.grad.copy_((torch.randn(n, device=dev()) * 3).bfloat16())
            ranks[2].grad[n - 5] = float("inf")      # lands in the last rank's slice
            want = sum(k.grad.float() for k in ranks)
        for k in ranks:
            cu().signal(f_ptrs, G, F_ARA, k.r, k.step)
        for k in ranks:
            cu().grad_allreduce(torch.bfloat16, g_ptrs, 0, n, G, k.r, k.flags[F_ARA:], f_ptrs, F_ARB, F_FOUND, k.step,
                                1, 0, k.counters[48:], 7)
        for k, hp in zip(ranks, hps):
            cu().wait_flags(k.flags[F_ARB:], G, k.step, 1, 0, k.flags[F_FOUND:], hp.buf)
        cu().check_status()
        for k, hp in zip(ranks, hps):
            got = k.grad.float()
            fin = torch.isfinite(want)
            torch.testing.assert_close(got[fin], want[fin], rtol=1e-2, atol=5e-2)
            assert float(hp.buf[HP.FOUND_INF]) == float(rnd)
            assert k.flags[F_FOUND:F_FOUND + G].abs().sum().item() == 0      # words cleared for the next step
            assert k.flags[F_ARB:F_ARB + G].tolist() == [rnd + 1] * G


def test_bounded_wait_times_out_with_status_and_context_survives():
    """A flag that nothing sets: the pull kernel gives up after its time budget, writes a status
    word, produces zeros, and later launches on the same context still work."""
    G, b, D = 2, 4, 64
    k = Rank(0, G, 8, D, 8)
    k.step.fill_(5)
    k.flags[F_RS] = 5                     # rank 0's flag is there, rank 1's never arrives
    d_ptrs = cu().ptr_array([k.dXp.data_ptr(), k.dXp.data_ptr()])
    de = torch.full((b, D), 3.0, device=dev())
    cu().rs_pull(d_ptrs, G, 0, b, D, de, k.flags[F_RS:], k.step, 0.0, k.rng, 5)
    torch.cuda.synchronize()
    with pytest.raises(cu().KernelError, match="timed out"):
        cu().check_status()
    assert float(de.abs().max()) == 0.0
    cu().check_status()                   # status was cleared by the failed check
    x = torch.ones(16, device=dev())
    assert float((x * 2).sum()) == 32.0   # the context is still usable


def test_sharded_adamw_emulated_matches_full_adamw():
    """Reduce-scatter + AdamW on each rank's slice + parameter push equals all-reduce + full AdamW."""
    from renee_b200.parallel.fused import F_ARC
    G, n, n_decay = 4, 8 * 1031, 8 * 500
    torch.manual_seed(2)
    ranks = [Rank(r, G, 8, 8, n) for r in range(G)]
    p0 = torch.randn(n, device=dev())
    m0, v0 = torch.rand(n, device=dev()) * 0.1, torch.rand(n, device=dev()) * 0.01
    st = []
    for k in ranks:
        k.grad.copy_((torch.randn(n, device=dev()) * 64).bfloat16())
        hp = HyperParams(dev(), init_scale=64.0)
        hp.buf[HP.LR_ENC] = 1e-2
        hp.buf[HP.ADAM_STEP] = 2
        st.append(dict(p32=p0.clone(), m=m0.clone(), v=v0.clone(), p16=p0.bfloat16(), hp=hp,
                       gsum=torch.zeros(n // G + 64, device=dev())))
    gsum_all = sum(k.grad.float() for k in ranks)
    rp, rm, rv = p0.clone(), m0.clone(), v0.clone()
    ref.adamw_step(rp, rm, rv, gsum_all, None, 1e-2, 0.9, 0.999, 1e-6, 0.01, n_decay, 3.0, (1 / 64.0) / G, 0.0)
    g_ptrs = cu().ptr_array([k.grad.data_ptr() for k in ranks])
    f_ptrs = cu().ptr_array([k.flags.data_ptr() for k in ranks])
    p_ptrs = cu().ptr_array([s["p16"].data_ptr() for s in st])
    for k in ranks:
        cu().signal(f_ptrs, G, F_ARA, k.r, k.step)
    for k, s in zip(ranks, st):
        cu().grad_reduce_scatter(torch.bfloat16, g_ptrs, n, G, k.r, k.flags[F_ARA:], k.step, s["gsum"], f_ptrs, F_ARB,
                                 F_FOUND, k.counters[48:], 5)
    for k, s in zip(ranks, st):
        cu().wait_flags(k.flags[F_ARB:], G, k.step, 1, 0, k.flags[F_FOUND:], s["hp"].buf)
    for k, s in zip(ranks, st):
        cu().adamw_shard_push(torch.bfloat16, s["p32"], s["m"], s["v"], s["gsum"], p_ptrs, n, n_decay, G, k.r, s["hp"].buf,
                              0.9, 0.999, 1e-6, 0.01, 1.0 / G, f_ptrs, F_ARC, k.step, k.counters[52:], 5)
    for k in ranks:
        cu().wait_flags(k.flags[F_ARC:], G, k.step, 1, 0, None, None)
    cu().check_status()
    per = ((n // 8) + G - 1) // G * 8
    for k, s in zip(ranks, st):
        lo, hi = min(n, per * k.r), min(n, per * (k.r + 1))
        torch.testing.assert_close(s["p32"][lo:hi], rp[lo:hi], rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(s["m"][lo:hi], rm[lo:hi], rtol=1e-5, atol=1e-7)
        torch.testing.assert_close(s["v"][lo:hi], rv[lo:hi], rtol=1e-5, atol=1e-7)
        assert torch.equal(s["p32"][:lo], p0[:lo]) and torch.equal(s["p32"][hi:], p0[hi:])   # other slices untouched
        torch.testing.assert_close(s["p16"].float(), rp, rtol=1e-2, atol=1e-2)                  # every slice arrived
        assert k.flags[F_ARC:F_ARC + G].tolist() == [1] * G


def test_bucketed_reduce_scatter_emulated_three_buckets():
    """The overlapped form of the sharded optimizer: the flat gradient is reduced bucket by bucket, every rank
    owning 1/G of EACH bucket, each bucket as soon as all ranks have reported the stage that completes it; then
    one AdamW launch over all of a rank's ranges.  Equals all-reduce + full AdamW."""
    from renee_b200.parallel.fused import F_ARC
    G, n, n_decay = 4, 8 * 1200, 8 * 700
    torch.manual_seed(3)
    ranks = [Rank(r, G, 8, 8, n) for r in range(G)]
    buckets = [(1, 8 * 700, 8 * 1100), (2, 8 * 300, 8 * 700), (3, 0, 8 * 300), (3, 8 * 1100, n)]   # (stage, lo, hi)
    p0 = torch.randn(n, device=dev())
    m0, v0 = torch.rand(n, device=dev()) * 0.1, torch.rand(n, device=dev()) * 0.01
    st = []
    for k in ranks:
        k.grad.copy_((torch.randn(n, device=dev()) * 64).bfloat16())
        hp = HyperParams(dev(), init_scale=64.0)
        hp.buf[HP.LR_ENC] = 1e-2
        hp.buf[HP.ADAM_STEP] = 2
        st.append(dict(p32=p0.clone(), m=m0.clone(), v=v0.clone(), p16=p0.bfloat16(), hp=hp,
                       gsum=torch.zeros(n // G + 256, device=dev())))
    gsum_all = sum(k.grad.float() for k in ranks)
    rp, rm, rv = p0.clone(), m0.clone(), v0.clone()
    ref.adamw_step(rp, rm, rv, gsum_all, None, 1e-2, 0.9, 0.999, 1e-6, 0.01, n_decay, 3.0, (1 / 64.0) / G, 0.0)

    def plan(r):
        out, g0 = [], 0
        for stage, lo, hi in buckets:
            n_vec = (hi - lo) // 8
            per = (n_vec + G - 1) // G
            a, b = lo // 8 + min(n_vec, per * r), lo // 8 + min(n_vec, per * (r + 1))
            if b > a:
                out.append((stage, a, b, g0))
                g0 += b - a
        return out

    g_ptrs = cu().ptr_array([k.grad.data_ptr() for k in ranks])
    f_ptrs = cu().ptr_array([k.flags.data_ptr() for k in ranks])
    p_ptrs = cu().ptr_array([s["p16"].data_ptr() for s in st])
    for stage in (1, 2, 3):
        for k in ranks:                                   # every emulated rank reports the stage ...
            cu().signal(f_ptrs, G, F_ARA, k.r, k.step, 32, stage)
        for k, s in zip(ranks, st):                       # ... then every rank reduces its part of the stage's buckets
            mine = [b for b in plan(k.r) if b[0] == stage]
            for i, (_, a, b, g0) in enumerate(mine):
                final = stage == 3 and i == len(mine) - 1
                cu().grad_reduce_scatter_range(torch.bfloat16, g_ptrs, a, b, G, k.r, k.flags[F_ARA:], k.step, 32, stage,
                                               s["gsum"][g0 * 8:], f_ptrs, F_ARB if final else -1, F_FOUND,
                                               k.counters[48:], 3)
    for k, s in zip(ranks, st):
        cu().wait_flags(k.flags[F_ARB:], G, k.step, 1, 0, k.flags[F_FOUND:], s["hp"].buf)
    for k, s in zip(ranks, st):
        cu().adamw_ranges_push(torch.bfloat16, s["p32"], s["m"], s["v"], s["gsum"], p_ptrs,
                               [(a, b, g0) for _, a, b, g0 in plan(k.r)], n_decay, G, k.r, s["hp"].buf, 0.9, 0.999, 1e-6,
                               0.01, 1.0 / G, f_ptrs, F_ARC, k.step, k.counters[52:], 3)
    for k in ranks:
        cu().wait_flags(k.flags[F_ARC:], G, k.step, 1, 0, None, None)
    cu().check_status()
    for k, s in zip(ranks, st):
        own = torch.zeros(n, dtype=torch.bool, device=dev())
        for _, a, b, _ in plan(k.r):
            own[a * 8: b * 8] = True
        torch.testing.assert_close(s["p32"][own], rp[own], rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(s["m"][own], rm[own], rtol=1e-5, atol=1e-7)
        assert torch.equal(s["p32"][~own], p0[~own])                                      # other ranks' parts untouched
        torch.testing.assert_close(s["p16"].float(), rp, rtol=1e-2, atol=1e-2)           # every part arrived
        assert float(s["hp"].buf[HP.FOUND_INF]) == 0.0
