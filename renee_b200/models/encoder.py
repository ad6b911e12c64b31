"""DistilBERT-style text encoder with HuggingFace-compatible parameter names.

The reference loads ``transformers.AutoModel`` (main.py:126-129) and wraps it in
``TransformerInputLayer`` (dl_base.py:121-141), which mean-pools the last hidden state under the
attention mask.  This module is an own implementation of the same architecture so that

* its ``state_dict`` keys equal HF DistilBERT's (``embeddings.word_embeddings.weight``,
  ``transformer.layer.N.attention.q_lin.weight`` ...), which keeps the reference's checkpoint
  layout ``embed.0.transformer.<hf-key>`` loadable in both directions;
* the fused engine (``renee_b200.models.flat_encoder``) can address all parameters as views of
  one flat buffer.

Architecture (checked against transformers' DistilBERT): word + learned position embeddings →
LayerNorm(eps 1e-12) → dropout; each block ``h = LN(x + drop(out_lin(attn(x))))`` then
``LN(h + drop(lin2(gelu(lin1(h)))))``; exact-erf GELU; no token types, no pooler.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class EncoderConfig:
    vocab_size: int = 30522
    max_position_embeddings: int = 512
    dim: int = 768
    n_layers: int = 6
    n_heads: int = 12
    hidden_dim: int = 3072
    dropout: float = 0.1
    attention_dropout: float = 0.1
    layer_norm_eps: float = 1e-12
    initializer_range: float = 0.02
    pad_token_id: int = 0
    attn_output_dropout: float = 0.0   # BERT/RoBERTa drop the attention output projection; DistilBERT does not

    @property
    def hidden_size(self) -> int:  # HF alias used by the reference (main.py:149,152)
        return self.dim

    def to_dict(self) -> dict:
        return asdict(self)


ENCODER_PRESETS = {
    # name fragments → config; any DistilBERT-family checkpoint name maps to the base shape
    "distilbert": EncoderConfig(),
    "tiny": EncoderConfig(dim=128, n_layers=2, n_heads=2, hidden_dim=512),
    "minilm-l6": EncoderConfig(dim=384, n_layers=6, n_heads=12, hidden_dim=1536, attn_output_dropout=0.1),
    "minilm-l3": EncoderConfig(dim=384, n_layers=3, n_heads=12, hidden_dim=1536, attn_output_dropout=0.1),
    "distilroberta": EncoderConfig(vocab_size=50265, max_position_embeddings=512, layer_norm_eps=1e-5,
                                   attn_output_dropout=0.1, pad_token_id=1),
    "roberta-large": EncoderConfig(vocab_size=50265, max_position_embeddings=512, dim=1024, n_layers=24,
                                   n_heads=16, hidden_dim=4096, layer_norm_eps=1e-5, attn_output_dropout=0.1,
                                   pad_token_id=1),
}


def config_from_name(name: str) -> EncoderConfig:
    """Map a ``--tf`` model id to an architecture.  Weights are random-init unless a state dict is
    loaded; there is no hub access in an offline deployment."""
    low = name.lower()
    if low in ENCODER_PRESETS:
        return ENCODER_PRESETS[low]
    if "roberta-large" in low:
        return ENCODER_PRESETS["roberta-large"]
    if "distilroberta" in low:
        return ENCODER_PRESETS["distilroberta"]
    if "minilm-l3" in low or "minilm_l3" in low:
        return ENCODER_PRESETS["minilm-l3"]
    if "minilm" in low:
        return ENCODER_PRESETS["minilm-l6"]
    if "tiny" in low:
        return ENCODER_PRESETS["tiny"]
    return ENCODER_PRESETS["distilbert"]


class Embeddings(nn.Module):
    def __init__(self, cfg: EncoderConfig):
        super().__init__()
        self.word_embeddings = nn.Embedding(cfg.vocab_size, cfg.dim, padding_idx=cfg.pad_token_id)
        self.position_embeddings = nn.Embedding(cfg.max_position_embeddings, cfg.dim)
        self.LayerNorm = nn.LayerNorm(cfg.dim, eps=cfg.layer_norm_eps)
        self.dropout = nn.Dropout(cfg.dropout)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        S = input_ids.size(1)
        pos = torch.arange(S, device=input_ids.device)
        x = self.word_embeddings(input_ids.long()) + self.position_embeddings(pos)[None]
        return self.dropout(self.LayerNorm(x))


class SelfAttention(nn.Module):
    def __init__(self, cfg: EncoderConfig):
        super().__init__()
        self.n_heads = cfg.n_heads
        self.dim = cfg.dim
        self.p = cfg.attention_dropout
        self.q_lin = nn.Linear(cfg.dim, cfg.dim)
        self.k_lin = nn.Linear(cfg.dim, cfg.dim)
        self.v_lin = nn.Linear(cfg.dim, cfg.dim)
        self.out_lin = nn.Linear(cfg.dim, cfg.dim)

    def forward(self, x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        b, S, _ = x.shape
        hd = self.dim // self.n_heads

        def split(t):
            return t.view(b, S, self.n_heads, hd).transpose(1, 2)

        q, k, v = split(self.q_lin(x)), split(self.k_lin(x)), split(self.v_lin(x))
        scores = torch.matmul(q, k.transpose(-1, -2)) / math.sqrt(hd)
        scores = scores.masked_fill(mask[:, None, None, :] == 0, torch.finfo(scores.dtype).min)
        w = F.dropout(torch.softmax(scores, dim=-1), self.p, self.training)
        ctx = torch.matmul(w, v).transpose(1, 2).reshape(b, S, self.dim)
        return self.out_lin(ctx)


class FFN(nn.Module):
    def __init__(self, cfg: EncoderConfig):
        super().__init__()
        self.lin1 = nn.Linear(cfg.dim, cfg.hidden_dim)
        self.lin2 = nn.Linear(cfg.hidden_dim, cfg.dim)
        self.dropout = nn.Dropout(cfg.dropout)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.dropout(self.lin2(F.gelu(self.lin1(x))))


class TransformerBlock(nn.Module):
    def __init__(self, cfg: EncoderConfig):
        super().__init__()
        self.attention = SelfAttention(cfg)
        self.sa_layer_norm = nn.LayerNorm(cfg.dim, eps=cfg.layer_norm_eps)
        self.ffn = FFN(cfg)
        self.output_layer_norm = nn.LayerNorm(cfg.dim, eps=cfg.layer_norm_eps)
        self.attn_dropout = nn.Dropout(cfg.attn_output_dropout)

    def forward(self, x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        h = self.sa_layer_norm(self.attn_dropout(self.attention(x, mask)) + x)
        return self.output_layer_norm(self.ffn(h) + h)


class _Layers(nn.Module):
    def __init__(self, cfg: EncoderConfig):
        super().__init__()
        self.layer = nn.ModuleList([TransformerBlock(cfg) for _ in range(cfg.n_layers)])


class DistilEncoder(nn.Module):
    """``forward(input_ids, attention_mask) -> {'last_hidden_state': [b, S, dim]}``."""

    def __init__(self, cfg: EncoderConfig):
        super().__init__()
        self.config = cfg
        self.embeddings = Embeddings(cfg)
        self.transformer = _Layers(cfg)
        self.apply(self._init)

    def _init(self, m: nn.Module) -> None:
        std = self.config.initializer_range
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, 0.0, std)
            nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, 0.0, std)
            if m.padding_idx is not None:
                with torch.no_grad():
                    m.weight[m.padding_idx].zero_()
        elif isinstance(m, nn.LayerNorm):
            nn.init.ones_(m.weight)
            nn.init.zeros_(m.bias)

    def forward(self, input_ids: torch.Tensor, attention_mask: torch.Tensor) -> dict:
        x = self.embeddings(input_ids)
        for blk in self.transformer.layer:
            x = blk(x, attention_mask)
        return {"last_hidden_state": x}


def convert_bert_state_dict(sd: dict, roberta: bool = False) -> dict:
    """Map a HF BERT / RoBERTa / MiniLM (BERT-architecture) encoder state dict onto this module's
    DistilBERT-style names.  The block math is identical (post-LayerNorm, erf GELU); the differences are
    absorbed exactly for single-segment, right-padded inputs:

    * ``token_type_embeddings[0]`` is added to every position embedding;
    * RoBERTa numbers real tokens from ``padding_idx + 1 = 2``, so its position table is shifted by two.

    (The reference takes any ``AutoModel``, main.py:126-129; its recipes use DistilBERT, DistilRoBERTa,
    RoBERTa-large and MiniLM, scripts/train_commands.md.)"""
    g = lambda k: sd[k] if k in sd else sd["bert." + k] if ("bert." + k) in sd else sd["roberta." + k]
    out = {}
    pos = g("embeddings.position_embeddings.weight").clone().float()
    tt = g("embeddings.token_type_embeddings.weight")[0].float()
    if roberta:
        pos = pos[2:]
    out["embeddings.word_embeddings.weight"] = g("embeddings.word_embeddings.weight")
    out["embeddings.position_embeddings.weight"] = pos + tt[None]
    out["embeddings.LayerNorm.weight"] = g("embeddings.LayerNorm.weight")
    out["embeddings.LayerNorm.bias"] = g("embeddings.LayerNorm.bias")
    l = 0
    while True:
        src = f"encoder.layer.{l}."
        try:
            g(src + "attention.self.query.weight")
        except KeyError:
            break
        dst = f"transformer.layer.{l}."
        for a, b in (("attention.self.query", "attention.q_lin"), ("attention.self.key", "attention.k_lin"),
                     ("attention.self.value", "attention.v_lin"), ("attention.output.dense", "attention.out_lin"),
                     ("attention.output.LayerNorm", "sa_layer_norm"), ("intermediate.dense", "ffn.lin1"),
                     ("output.dense", "ffn.lin2"), ("output.LayerNorm", "output_layer_norm")):
            for kind in ("weight", "bias"):
                out[dst + b + "." + kind] = g(src + a + "." + kind)
        l += 1
    return out


def strip_ngame_prefix(state_dict: dict) -> dict:
    """NGAME-pretrained encoders store keys under
    ``embedding_labels.encoder.transformer.0.auto_model.`` (reference main.py:133-145)."""
    pre = "embedding_labels.encoder.transformer.0.auto_model."
    return {k.replace(pre, ""): v for k, v in state_dict.items()}


class TransformerInputLayer(nn.Module):
    """Encoder + pooling.  ``pooling='mean'`` is the reference's mask-weighted mean in fp32
    (dl_base.py:131-141); ``'cls'`` takes the first token's hidden state."""

    def __init__(self, transformer: nn.Module, pooling: str = "mean"):
        super().__init__()
        if pooling not in ("mean", "cls"):
            raise ValueError("pooling must be 'mean' or 'cls'")
        self.transformer = transformer
        self.pooling = pooling

    def forward(self, data: dict) -> torch.Tensor:
        h = self.transformer(input_ids=data["input_ids"], attention_mask=data["attention_mask"])["last_hidden_state"]
        if self.pooling == "cls":
            return h[:, 0].float().contiguous()
        m = data["attention_mask"].unsqueeze(-1).expand(h.size()).float()
        return ((h.float() * m).sum(1) / m.sum(1).clamp(min=1e-9)).contiguous()


class FP32Linear(nn.Module):
    """Optional bottleneck ``hidden -> D`` computed in fp32 regardless of autocast.  Parameter
    names ``transformer_weight``/``transformer_bias`` are kept so that they fall in the encoder's
    Adam group rather than the classifier's SGD group (reference dl_base.py:92-118, 219-226)."""

    def __init__(self, input_size: int, output_size: int, bias: bool = True):
        super().__init__()
        self.input_size, self.output_size = input_size, output_size
        self.transformer_weight = nn.Parameter(torch.empty(output_size, input_size))
        if bias:
            self.transformer_bias = nn.Parameter(torch.empty(output_size))
        else:
            self.register_parameter("transformer_bias", None)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        stdv = 1.0 / math.sqrt(self.input_size)
        with torch.no_grad():
            self.transformer_weight.uniform_(-stdv, stdv)
            if self.transformer_bias is not None:
                self.transformer_bias.uniform_(-stdv, stdv)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        with torch.autocast(device_type=x.device.type, enabled=False):
            return F.linear(x.float(), self.transformer_weight, self.transformer_bias)
