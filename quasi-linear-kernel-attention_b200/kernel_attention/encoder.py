"""A plain pre-LN transformer encoder whose attention is one of the additive kernels, for end-to-end
latency and peak-memory measurements of the operators (defaults: 12 layers, hidden 768,
12 heads of 64, MLP 3072 with GELU, rotary positions, vocabulary 30528, fp32, random weights).

The reference has no such encoder of its own; the block structure follows its pre-LN `EncoderBlock`
(Experiments/kernel_attention/vision_transformer.py:59-77) and the rotary kernel attention of
Experiments/kernel_attention/nomic.py:9-30. Attention kernels: "add_laplace", "add_riesz", "add_bump"
(this library) or "softmax" (torch scaled_dot_product_attention, for comparison).

    python quasi-linear-kernel-attention_b200/kernel_attention/encoder.py [--batch 2 --seq 8192 --kernel add_laplace]
"""

import argparse
import math
import os
import sys
import time

import torch
import torch.nn as nn
import torch.nn.functional as F


def rotary(x, base=10000.0):
    """Rotary position embedding on (B, H, S, Dh), pairs (i, i + Dh/2)."""
    B, H, S, Dh = x.shape
    half = Dh // 2
    freq = base ** (-torch.arange(half, device=x.device, dtype=torch.float32) / half)
    ang = torch.arange(S, device=x.device, dtype=torch.float32)[:, None] * freq[None, :]      # (S, half)
    cos, sin = ang.cos()[None, None], ang.sin()[None, None]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1)


class Block(nn.Module):
    def __init__(self, hidden, heads, mlp, kernel, tau):
        super().__init__()
        self.heads, self.kernel, self.tau = heads, kernel, tau
        self.ln1, self.ln2 = nn.LayerNorm(hidden), nn.LayerNorm(hidden)
        self.qkv, self.proj = nn.Linear(hidden, 3 * hidden), nn.Linear(hidden, hidden)
        self.fc1, self.fc2 = nn.Linear(hidden, mlp), nn.Linear(mlp, hidden)

    def attend(self, x, keep):
        B, S, Hd = x.shape
        q, k, v = self.qkv(x).view(B, S, 3, self.heads, Hd // self.heads).permute(2, 0, 3, 1, 4)   # 3 x (B, H, S, Dh)
        q, k = rotary(q), rotary(k)
        if self.kernel == "softmax":
            mask = None if keep is None else keep[:, None, None, :]
            o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
        else:
            from kernel_attention.attention import attention
            o = attention(q.contiguous(), k.contiguous(), v.contiguous(), self.kernel, self.tau, keep)
        return self.proj(o.transpose(1, 2).reshape(B, S, Hd))

    def forward(self, x, keep=None):
        x = x + self.attend(self.ln1(x), keep)
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x))))


class Encoder(nn.Module):
    def __init__(self, kernel="add_laplace", tau=None, layers=12, hidden=768, heads=12, mlp=3072, vocab=30528):
        super().__init__()
        from kernel_attention.attention import TAU
        tau = TAU.get(kernel, 1.0) if tau is None else tau
        self.embed = nn.Embedding(vocab, hidden)
        self.blocks = nn.ModuleList(Block(hidden, heads, mlp, kernel, tau) for _ in range(layers))
        self.ln = nn.LayerNorm(hidden)

    @torch.no_grad()
    def forward(self, ids, keep=None):
        x = self.embed(ids)
        for blk in self.blocks:
            x = blk(x, keep)
        return self.ln(x)


def measure(kernel, batch, seq, layers=12, reps=3, seed=0):
    """(latency in ms, peak memory in MiB) of one forward pass on cuda:0, fp32, random weights and token ids."""
    torch.manual_seed(seed)
    dev = torch.device("cuda", 0)
    model = Encoder(kernel, layers=layers).to(dev).eval()
    ids = torch.randint(0, 30528, (batch, seq), device=dev)
    model(ids)
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        model(ids)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps, (torch.cuda.max_memory_allocated() - base) / 2 ** 20


if __name__ == "__main__":
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, here)
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--kernel", default="add_laplace")
    a = ap.parse_args()
    ms, mib = measure(a.kernel, a.batch, a.seq, a.layers)
    print(f'{{"kernel": "{a.kernel}", "batch": {a.batch}, "seq": {a.seq}, "layers": {a.layers}, "latency_ms": {ms:.3f}, "peak_mib": {mib:.1f}}}')
