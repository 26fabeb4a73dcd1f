"""Transformer encoders/decoders for the language-model benchmarks:
BERT-large (masked LM, 24 layers, hidden 1024, 16 heads, FFN 4096, vocab
30522, ~340 M parameters) and GPT-2 medium (causal LM, 24 layers, d_model
1024, 16 heads, FFN 4096, vocab 50257, context 1024, ~355 M parameters).
Attention uses torch.nn.functional.scaled_dot_product_attention.
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class SelfAttention(nn.Module):
    def __init__(self, d_model, n_heads, causal):
        super().__init__()
        self.n_heads = n_heads
        self.causal = causal
        self.qkv = nn.Linear(d_model, 3 * d_model)
        self.proj = nn.Linear(d_model, d_model)

    def forward(self, x):
        b, s, d = x.shape
        q, k, v = self.qkv(x).view(b, s, 3, self.n_heads, d // self.n_heads).unbind(2)
        y = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2),
                                           v.transpose(1, 2), is_causal=self.causal)
        return self.proj(y.transpose(1, 2).reshape(b, s, d))


class Block(nn.Module):
    def __init__(self, d_model, n_heads, d_ff, causal, pre_norm):
        super().__init__()
        self.pre_norm = pre_norm
        self.ln1 = nn.LayerNorm(d_model)
        self.attn = SelfAttention(d_model, n_heads, causal)
        self.ln2 = nn.LayerNorm(d_model)
        self.fc1 = nn.Linear(d_model, d_ff)
        self.fc2 = nn.Linear(d_ff, d_model)

    def forward(self, x):
        if self.pre_norm:  # GPT-2
            x = x + self.attn(self.ln1(x))
            return x + self.fc2(F.gelu(self.fc1(self.ln2(x))))
        x = self.ln1(x + self.attn(x))  # BERT
        return self.ln2(x + self.fc2(F.gelu(self.fc1(x))))


class TransformerLM(nn.Module):
    def __init__(self, vocab, max_len, d_model, n_layers, n_heads, d_ff, causal,
                 segments=0):
        super().__init__()
        self.causal = causal
        self.tok = nn.Embedding(vocab, d_model)
        self.pos = nn.Embedding(max_len, d_model)
        self.seg = nn.Embedding(segments, d_model) if segments else None
        self.emb_ln = None if causal else nn.LayerNorm(d_model)
        self.blocks = nn.ModuleList(
            [Block(d_model, n_heads, d_ff, causal, pre_norm=causal) for _ in range(n_layers)])
        self.final_ln = nn.LayerNorm(d_model) if causal else None
        if not causal:  # BERT MLM head: dense + gelu + LN, decoder tied to embeddings
            self.head_fc = nn.Linear(d_model, d_model)
            self.head_ln = nn.LayerNorm(d_model)
            self.head_bias = nn.Parameter(torch.zeros(vocab))
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
        if isinstance(m, nn.Linear) and m.bias is not None:
            nn.init.zeros_(m.bias)

    def forward(self, ids):
        b, s = ids.shape
        x = self.tok(ids) + self.pos(torch.arange(s, device=ids.device))
        if self.seg is not None:
            x = x + self.seg.weight[0]
        if self.emb_ln is not None:
            x = self.emb_ln(x)
        for blk in self.blocks:
            x = blk(x)
        if self.causal:
            return F.linear(self.final_ln(x), self.tok.weight)
        h = self.head_ln(F.gelu(self.head_fc(x)))
        return F.linear(h, self.tok.weight, self.head_bias)


def bert_large(vocab=30522, max_len=512):
    return TransformerLM(vocab, max_len, 1024, 24, 16, 4096, causal=False, segments=2)


def gpt2_medium(vocab=50257, max_len=1024):
    return TransformerLM(vocab, max_len, 1024, 24, 16, 4096, causal=True)


def tiny_lm(causal=True, vocab=128, max_len=32):
    return TransformerLM(vocab, max_len, 32, 2, 2, 64, causal=causal,
                         segments=0 if causal else 2)
