"""The hand-written encoder forward/backward equals autograd through the module implementation."""
import functools

import torch

from renee_b200 import ops
from renee_b200.models.encoder import DistilEncoder, EncoderConfig, FP32Linear, TransformerInputLayer
from renee_b200.models.flat_encoder import FlatEncoder
from renee_b200.ops import reference as ref


_close = functools.partial(torch.testing.assert_close, rtol=1e-4, atol=1e-5, check_dtype=False)


def _cfg(p=0.0):
    return EncoderConfig(vocab_size=200, max_position_embeddings=16, dim=128, n_layers=2, n_heads=2,
                         hidden_dim=256, dropout=p, attention_dropout=p)


def _inputs(b=5, S=12):
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(3, S + 1, (b,), generator=g)
    mask = (torch.arange(S)[None] < lens[:, None]).int()
    ids = torch.randint(1, 200, (b, S), generator=g).int() * mask
    return ids, mask


def _pair(pooling, bottleneck):
    cfg = _cfg()
    torch.manual_seed(1)
    mod = DistilEncoder(cfg).double()
    # non-trivial LayerNorm/bias values so that their gradients are exercised
    with torch.no_grad():
        for n, p in mod.named_parameters():
            if "bias" in n or "norm" in n.lower():
                p.add_(0.1 * torch.randn_like(p))
    wrap = TransformerInputLayer(mod, pooling)
    flat = FlatEncoder(cfg, "cpu", torch.float32, pooling, bottleneck, seed=3)
    flat.load_encoder_state_dict({k: v.float() for k, v in mod.state_dict().items()})
    return cfg, mod, wrap, flat


def _check(pooling, bottleneck):
    cfg, mod, wrap, flat = _pair(pooling, bottleneck)
    ids, mask = _inputs()
    mod.eval()
    e_ref = wrap({"input_ids": ids, "attention_mask": mask})
    if bottleneck:
        lin = FP32Linear(cfg.dim, bottleneck, bias=False).double()
        with torch.no_grad():
            lin.transformer_weight.copy_(flat.bottleneck_weight().double())
        e_ref = torch.nn.functional.linear(e_ref.double(), lin.transformer_weight)
    rng = ops.StepRNG(0)
    e = flat.forward(ids, mask, rng, train=True)
    torch.testing.assert_close(e.double(), e_ref.double(), rtol=2e-4, atol=2e-5)
    d = torch.randn(e.shape, generator=torch.Generator().manual_seed(5))
    e_ref.backward(d.double())
    flat.backward(d.clone())
    for n, p in mod.named_parameters():
        g = flat.view(flat.g, n)
        want = p.grad.float()
        if n == "embeddings.word_embeddings.weight":
            want = want.clone(); want[cfg.pad_token_id] = 0      # padding_idx gets no gradient
        if n == "embeddings.position_embeddings.weight" or "weight" in n or "bias" in n:
            torch.testing.assert_close(g, want, rtol=2e-3, atol=2e-5, msg=lambda m: f"{n}: {m}")
    if bottleneck:
        torch.testing.assert_close(flat.view(flat.g, "__bottleneck__.transformer_weight"),
                                   lin.transformer_weight.grad.float(), rtol=2e-3, atol=2e-5)


def test_mean_pool_no_bottleneck():
    _check("mean", 0)


def test_cls_pool_with_bottleneck():
    _check("cls", 64)


def test_flat_layout_groups_and_qkv_adjacency():
    cfg = _cfg()
    f = FlatEncoder(cfg, "cpu", torch.float32)
    for n, s in f.slots.items():
        nodecay = any(k in n for k in ("bias", "LayerNorm.bias", "LayerNorm.weight"))
        assert (s.offset >= f.n_decay) == nodecay, n
        assert s.offset % 128 == 0
    # block LayerNorm weights are decayed (name quirk of the reference's filter), embeddings.LayerNorm is not
    assert f.slots["transformer.layer.0.sa_layer_norm.weight"].offset < f.n_decay
    assert f.slots["embeddings.LayerNorm.weight"].offset >= f.n_decay
    w = f._qkv(f.p32, 1, "weight")
    assert torch.equal(w[: cfg.dim], f.view(f.p32, "transformer.layer.1.attention.q_lin.weight"))
    assert torch.equal(w[2 * cfg.dim:], f.view(f.p32, "transformer.layer.1.attention.v_lin.weight"))
    sd = f.encoder_state_dict()
    assert set(sd) == set(DistilEncoder(cfg).state_dict())


def test_dropout_ops_backward_matches_autograd_with_shared_mask():
    """The fused fwd/bwd pairs agree with autograd when both use the counter-based mask."""
    torch.manual_seed(0)
    T, H, p, seed = 24, 128, 0.3, 1234
    x = torch.randn(T, H, dtype=torch.float64, requires_grad=True)
    res = torch.randn(T, H, dtype=torch.float64, requires_grad=True)
    bias = torch.randn(H, dtype=torch.float64, requires_grad=True)
    gam = torch.randn(H, dtype=torch.float64, requires_grad=True)
    bet = torch.randn(H, dtype=torch.float64, requires_grad=True)
    m = ops.keep_mask(seed, 9, (T, H), p).double() / (1 - p)
    y_ref = torch.nn.functional.layer_norm(res + (x + bias) * m, (H,), gam, bet, 1e-12)
    dy = torch.randn(T, H, dtype=torch.float64)
    y_ref.backward(dy)
    y, pre, mean, rstd = ref.bias_dropout_add_ln_fwd(x.detach(), bias.detach(), res.detach(), gam.detach(),
                                                     bet.detach(), 1e-12, p, seed, 9)
    _close(y, y_ref.detach())
    dg, db, dbias = torch.zeros(H, dtype=torch.float64), torch.zeros(H, dtype=torch.float64), torch.zeros(H, dtype=torch.float64)
    d_pre, d_branch = ref.bias_dropout_add_ln_bwd(dy, pre, gam.detach(), mean, rstd, p, seed, 9, dg, db, dbias)
    _close(d_pre, res.grad)
    _close(d_branch, x.grad)
    _close(dg, gam.grad); _close(db, bet.grad)
    _close(dbias, bias.grad)


def test_attention_reference_backward_matches_autograd_with_dropout():
    torch.manual_seed(0)
    b, S, nh, H, p, seed = 3, 8, 2, 32, 0.25, 77
    qkv = torch.randn(b * S, 3 * H, dtype=torch.float64, requires_grad=True)
    bq = torch.randn(3 * H, dtype=torch.float64, requires_grad=True)
    mask = torch.ones(b, S, dtype=torch.int32); mask[0, 5:] = 0; mask[2, 2:] = 0
    hd = H // nh
    x = (qkv + bq).view(b, S, 3, nh, hd)
    q, k, v = [x[:, :, i].transpose(1, 2) for i in range(3)]
    s = (q @ k.transpose(-1, -2)) / hd ** 0.5
    s = s.masked_fill(mask[:, None, None, :] == 0, -1e30)
    pr = torch.softmax(s, -1)
    w = pr * ops.keep_mask(seed, 4, pr.shape, p).double() / (1 - p)
    ctx_ref = (w @ v).transpose(1, 2).reshape(b * S, H)
    d = torch.randn(b * S, H, dtype=torch.float64)
    ctx_ref.backward(d)
    ctx, probs = ref.attention_fwd(qkv.detach(), bq.detach(), mask, nh, p, seed, 4)
    _close(ctx, ctx_ref.detach())
    dqkv = ref.attention_bwd(d, qkv.detach(), bq.detach(), mask, probs, nh, p, seed, 4)
    _close(dqkv, qkv.grad)


def test_gelu_and_pool_backward():
    torch.manual_seed(0)
    x = torch.randn(10, 16, dtype=torch.float64, requires_grad=True)
    bias = torch.randn(16, dtype=torch.float64, requires_grad=True)
    a = torch.nn.functional.gelu(x + bias)
    da = torch.randn_like(a)
    a.backward(da)
    dbias = torch.zeros(16, dtype=torch.float64)
    dx = ref.bias_gelu_bwd(da, x.detach(), bias.detach(), dbias)
    _close(dx, x.grad); _close(dbias, bias.grad)
    h = torch.randn(3, 5, 8, dtype=torch.float64, requires_grad=True)
    mask = torch.tensor([[1, 1, 1, 0, 0], [1, 1, 1, 1, 1], [1, 0, 0, 0, 0]], dtype=torch.int32)
    for mode in ("mean", "cls"):
        h.grad = None
        e = ref.pool_fwd(h, mask, mode)
        de = torch.randn(3, 8, dtype=torch.float64)
        if mode == "mean":
            m = mask.unsqueeze(-1).double()
            ((h * m).sum(1) / m.sum(1)).backward(de)
        else:
            h[:, 0].backward(de)
        _close(ref.pool_bwd(de, mask, mode, 5, torch.float64), h.grad)


def test_bert_and_roberta_checkpoints_map_onto_the_engine():
    """A HF BERT / RoBERTa encoder imported through convert_bert_state_dict gives the same hidden states."""
    from transformers import BertConfig, BertModel, RobertaConfig, RobertaModel
    from renee_b200.models.encoder import convert_bert_state_dict
    ids, mask = _inputs(b=4, S=10)
    for roberta in (False, True):
        kw = dict(vocab_size=200, hidden_size=128, num_hidden_layers=2, num_attention_heads=2, intermediate_size=256,
                  max_position_embeddings=32, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
        torch.manual_seed(0)
        if roberta:
            hf = RobertaModel(RobertaConfig(pad_token_id=1, layer_norm_eps=1e-5, **kw), add_pooling_layer=False).eval()
            toks = torch.where(mask.bool(), ids.long().clamp(min=2), torch.ones_like(ids.long()))
        else:
            hf = BertModel(BertConfig(layer_norm_eps=1e-12, **kw), add_pooling_layer=False).eval()
            toks = ids.long()
        with torch.no_grad():
            want = hf(input_ids=toks, attention_mask=mask.long()).last_hidden_state
        cfg = EncoderConfig(vocab_size=200, max_position_embeddings=30 if roberta else 32, dim=128, n_layers=2, n_heads=2,
                            hidden_dim=256, dropout=0.0, attention_dropout=0.0, layer_norm_eps=1e-5 if roberta else 1e-12,
                            pad_token_id=1 if roberta else 0)
        mine = DistilEncoder(cfg).eval()
        mine.load_state_dict(convert_bert_state_dict(hf.state_dict(), roberta=roberta))
        with torch.no_grad():
            got = mine(toks.int(), mask)["last_hidden_state"]
        valid = mask.bool()
        torch.testing.assert_close(got[valid], want[valid], rtol=1e-4, atol=1e-4)
