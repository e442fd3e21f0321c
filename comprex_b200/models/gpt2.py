"""GPT-2 (decoder-only transformer with learned positions, pre-LayerNorm, GELU MLP,
tied input/output embedding).  ``gpt2_medium()`` is the 24-layer, d_model 1024,
16-head, FFN 4096, vocabulary 50257, context 1024 configuration (355 M parameters).
Attention uses ``scaled_dot_product_attention`` (library kernel).
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class Block(nn.Module):
    def __init__(self, d, heads, ffn):
        super().__init__()
        self.heads = heads
        self.ln1 = nn.LayerNorm(d)
        self.qkv = nn.Linear(d, 3 * d)
        self.proj = nn.Linear(d, d)
        self.ln2 = nn.LayerNorm(d)
        self.fc = nn.Linear(d, ffn)
        self.out = nn.Linear(ffn, d)

    def forward(self, x):
        b, t, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(b, t, 3, self.heads, d // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(b, t, d))
        return x + self.out(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))


class GPT2(nn.Module):
    def __init__(self, layers=24, d_model=1024, heads=16, ffn=4096, vocab=50257, ctx=1024):
        super().__init__()
        self.wte = nn.Embedding(vocab, d_model)
        self.wpe = nn.Embedding(ctx, d_model)
        self.blocks = nn.ModuleList(Block(d_model, heads, ffn) for _ in range(layers))
        self.ln_f = nn.LayerNorm(d_model)
        self.apply(self._init)
        for blk in self.blocks:
            nn.init.normal_(blk.proj.weight, std=0.02 / math.sqrt(2 * layers))
            nn.init.normal_(blk.out.weight, std=0.02 / math.sqrt(2 * layers))

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
            if isinstance(m, nn.Linear) and m.bias is not None:
                nn.init.zeros_(m.bias)

    def forward(self, idx, targets=None):
        b, t = idx.shape
        x = self.wte(idx) + self.wpe(torch.arange(t, device=idx.device))
        for blk in self.blocks:
            x = blk(x)
        logits = F.linear(self.ln_f(x), self.wte.weight)
        if targets is None:
            return logits
        return F.cross_entropy(logits.float().view(-1, logits.size(-1)), targets.view(-1))


def gpt2_medium():
    return GPT2(24, 1024, 16, 4096, 50257, 1024)


def gpt2_tiny(vocab=257, ctx=64):
    return GPT2(2, 64, 4, 128, vocab, ctx)
