"""UMT5-style text encoder (encoder stack only).

Pre-norm blocks of ``T5LayerNorm -> self-attention with per-layer relative position bias -> residual``
and ``T5LayerNorm -> gated-GELU feed-forward -> residual``; no absolute positions, no attention
scaling (folded into the initialisation), padding keys masked.  State-dict names follow the
reference's ``T5Encoder`` (token_embedding, blocks.N.{norm1,attn.{q,k,v,o},pos_embedding.embedding,
norm2,ffn.{gate.0,fc1,fc2}}, norm) so the published ``umt5-xxl`` encoder weights load by name
(reference: solar/backends/wan22/runtime/modeling/t5.py, WanTextEncoder in runtime/components.py:21-64).

``HashTokenizer`` is the offline stand-in used when no sentencepiece model file is configured: a
stable blake2 hash of whitespace-separated pieces into the vocabulary, pad id 0, eos id 1.
"""
from __future__ import annotations

import hashlib
import math
from dataclasses import dataclass
from typing import List, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class T5Config:
    vocab: int = 256384
    dim: int = 4096
    dim_attn: int = 4096
    dim_ffn: int = 10240
    num_heads: int = 64
    num_layers: int = 24
    num_buckets: int = 32
    max_distance: int = 128
    text_len: int = 512

    @classmethod
    def tiny(cls):
        return cls(vocab=512, dim=32, dim_attn=32, dim_ffn=64, num_heads=2, num_layers=2, text_len=8)


class T5LayerNorm(nn.Module):
    def __init__(self, dim, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        v = x.float().pow(2).mean(-1, keepdim=True)
        return (x.float() * torch.rsqrt(v + self.eps)).to(x.dtype) * self.weight


class RelativeBias(nn.Module):
    def __init__(self, buckets, heads, max_distance):
        super().__init__()
        self.buckets, self.max_distance = buckets, max_distance
        self.embedding = nn.Embedding(buckets, heads)

    def forward(self, lq, lk, device):
        rel = torch.arange(lk, device=device)[None, :] - torch.arange(lq, device=device)[:, None]
        nb = self.buckets // 2                       # bidirectional
        bucket = (rel > 0).long() * nb
        rel = rel.abs()
        exact = nb // 2
        large = exact + (torch.log(rel.float().clamp_min(1) / exact) / math.log(self.max_distance / exact)
                         * (nb - exact)).long()
        large = large.clamp_max(nb - 1)
        bucket = bucket + torch.where(rel < exact, rel, large)
        return self.embedding(bucket).permute(2, 0, 1).unsqueeze(0)       # [1, H, lq, lk]


class _Gate(nn.Sequential):
    def __init__(self, dim, dim_ffn):
        super().__init__(nn.Linear(dim, dim_ffn, bias=False), nn.GELU(approximate="tanh"))


class T5Block(nn.Module):
    def __init__(self, c: T5Config):
        super().__init__()
        self.h = c.num_heads
        self.norm1 = T5LayerNorm(c.dim)
        self.attn = nn.ModuleDict(dict(q=nn.Linear(c.dim, c.dim_attn, bias=False), k=nn.Linear(c.dim, c.dim_attn, bias=False),
                                       v=nn.Linear(c.dim, c.dim_attn, bias=False), o=nn.Linear(c.dim_attn, c.dim, bias=False)))
        self.pos_embedding = RelativeBias(c.num_buckets, c.num_heads, c.max_distance)
        self.norm2 = T5LayerNorm(c.dim)
        self.ffn = nn.ModuleDict(dict(gate=_Gate(c.dim, c.dim_ffn), fc1=nn.Linear(c.dim, c.dim_ffn, bias=False),
                                      fc2=nn.Linear(c.dim_ffn, c.dim, bias=False)))

    def forward(self, x, mask):
        B, L, _ = x.shape
        y = self.norm1(x)
        q, k, v = (self.attn[n](y).view(B, L, self.h, -1).transpose(1, 2) for n in "qkv")
        bias = self.pos_embedding(L, L, x.device).to(q.dtype)
        if mask is not None:
            bias = bias.masked_fill(~mask[:, None, None, :], torch.finfo(q.dtype).min)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=bias, scale=1.0)
        x = x + self.attn["o"](o.transpose(1, 2).reshape(B, L, -1))
        y = self.norm2(x)
        return x + self.ffn["fc2"](self.ffn["fc1"](y) * self.ffn["gate"](y))


class T5Encoder(nn.Module):
    def __init__(self, c: T5Config = T5Config()):
        super().__init__()
        self.cfg = c
        self.token_embedding = nn.Embedding(c.vocab, c.dim)
        self.blocks = nn.ModuleList([T5Block(c) for _ in range(c.num_layers)])
        self.norm = T5LayerNorm(c.dim)

    def forward(self, ids, mask=None):
        x = self.token_embedding(ids)
        for b in self.blocks:
            x = b(x, mask)
        return self.norm(x)


class HashTokenizer:
    def __init__(self, vocab: int, text_len: int):
        self.vocab, self.text_len = vocab, text_len

    def __call__(self, texts: Sequence[str]):
        ids = torch.zeros(len(texts), self.text_len, dtype=torch.long)
        mask = torch.zeros(len(texts), self.text_len, dtype=torch.bool)
        for i, t in enumerate(texts):
            toks: List[int] = [2 + int.from_bytes(hashlib.blake2s(p.encode(), digest_size=4).digest(), "little") % (self.vocab - 2)
                               for p in t.strip().split()][: self.text_len - 1] + [1]
            ids[i, :len(toks)] = torch.tensor(toks)
            mask[i, :len(toks)] = True
        return ids, mask


def clean_prompt(text: str) -> str:
    """HTML entities resolved (twice, as scraped captions need), whitespace runs collapsed, ends stripped."""
    import html
    import re

    return re.sub(r"\s+", " ", html.unescape(html.unescape(text))).strip()


class PromptTokenizer:
    """The published tokenizer directory behind the ``(ids, mask)`` contract: ``tokenizer.json`` through the
    ``tokenizers`` library when present, else ``spiece.model`` through sentencepiece.  Prompts are cleaned, cut to
    ``text_len - 1`` pieces, closed with the end-of-sequence id and padded with the pad id (reference:
    solar/backends/wan22/runtime/modeling/tokenizers.py:20-82, ``padding="max_length", truncation=True``)."""

    def __init__(self, directory, text_len: int, *, pad_id: int = 0, eos_id: int = 1):
        from pathlib import Path

        root = Path(directory)
        self.text_len, self.pad_id, self.eos_id = int(text_len), pad_id, eos_id
        if (root / "tokenizer.json").is_file():
            from tokenizers import Tokenizer

            tk = Tokenizer.from_file(str(root / "tokenizer.json"))
            tk.no_padding()
            tk.no_truncation()
            self._pieces = lambda text: tk.encode(text, add_special_tokens=False).ids
        elif (root / "spiece.model").is_file():
            import sentencepiece

            sp = sentencepiece.SentencePieceProcessor(model_file=str(root / "spiece.model"))
            self._pieces = lambda text: list(sp.encode(text))
        else:
            raise FileNotFoundError(f"{root} holds neither tokenizer.json nor spiece.model")

    def __call__(self, texts: Sequence[str]):
        ids = torch.full((len(texts), self.text_len), self.pad_id, dtype=torch.long)
        mask = torch.zeros(len(texts), self.text_len, dtype=torch.bool)
        for i, t in enumerate(texts):
            toks = [x for x in self._pieces(clean_prompt(t)) if x != self.eos_id][: self.text_len - 1] + [self.eos_id]
            ids[i, :len(toks)] = torch.tensor(toks)
            mask[i, :len(toks)] = True
        return ids, mask


class WanTextEncoder:
    """prompts -> [B, text_len, dim] with the positions past each prompt zeroed (what the DiT's text
    embedding consumes)."""

    def __init__(self, cfg: T5Config = T5Config(), device="cpu", dtype=torch.bfloat16, tokenizer=None, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.model = T5Encoder(cfg)
        for p in self.model.parameters():
            if p.dim() > 1:
                with torch.no_grad():
                    p.copy_(torch.randn(p.shape, generator=g) * (1.0 / math.sqrt(p.shape[-1])))
        self.model = self.model.to(device=device, dtype=dtype).eval().requires_grad_(False)
        self.tok = tokenizer or HashTokenizer(cfg.vocab, cfg.text_len)
        self.device = torch.device(device)

    @classmethod
    def from_released(cls, weights, tokenizer_dir, *, cfg: T5Config = T5Config(), device="cpu", dtype=torch.bfloat16):
        """The published encoder file (``models_t5_umt5-xxl-enc-bf16.pth``: a plain state dict under the names of this
        module) loaded strictly, with the published tokenizer directory (reference: WanTextEncoder,
        solar/backends/wan22/runtime/components.py:21-64)."""
        self = cls.__new__(cls)
        with torch.device("meta"):
            model = T5Encoder(cfg)
        state = torch.load(str(weights), map_location="cpu", weights_only=True, mmap=True)
        result = model.load_state_dict(state, strict=True, assign=True)
        if result.missing_keys or result.unexpected_keys or any(p.is_meta for p in model.parameters()):
            raise ValueError(f"text-encoder checkpoint {weights} does not match the architecture")
        self.model = model.to(device=device, dtype=dtype).eval().requires_grad_(False)
        self.tok = PromptTokenizer(tokenizer_dir, cfg.text_len)
        self.device = torch.device(device)
        return self

    @torch.no_grad()
    def __call__(self, prompts: Sequence[str]):
        ids, mask = self.tok(prompts)
        ids, mask = ids.to(self.device), mask.to(self.device)
        out = self.model(ids, mask)
        return out * mask.unsqueeze(-1).to(out.dtype)
