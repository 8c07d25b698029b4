"""A nanochat-shaped language model whose attention blocks are DISM layers (hard path).

Plain torch everywhere except the sequence mixer: bias-free q/k/v/output projections, rotary position
embedding (base 100000) and a parameter-free RMS norm on q and k, pre-norm residual blocks, a 4x MLP with
squared ReLU, untied embedding and unembedding (the shape of the reference's nanochat GPT:
nanochat/nanochat/gpt.py:42-43,77-80,101-102,142-150,161-166,284-291).  The mixer replaces the attention
call (gpt.py:109-130) by `voc_dism` and adds what the reference's DISM module adds per layer: readout
projections sq/sk with SiLU (dism_v3/python/flash_dism/module.py:118-119,151-159), two codebooks [H,V,D]
initialised silu(N(0,1)) and a per-head log_sel_tau ~ U(-4,4) whose softplus is the weight coefficient
(module.py:125-131,376-380).  Every sequence runs hard: the operator's gradient reaches the model through
sq, sk, v and tau, as in the reference's hard training rows.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F


def rms(x, eps=1e-6):
    return x * torch.rsqrt(x.float().square().mean(-1, keepdim=True) + eps).to(x.dtype)


def rotary(x, cos, sin):
    """x [B,N,H,D]; cos, sin [N,1,D/2]."""
    a, b = x[..., : x.size(-1) // 2], x[..., x.size(-1) // 2:]
    return torch.cat((a * cos + b * sin, b * cos - a * sin), -1)


class DismLayer(nn.Module):
    def __init__(self, width, heads, head_dim, readout_dim=32, vocab_size=512):
        super().__init__()
        self.heads, self.head_dim, self.readout_dim = heads, head_dim, readout_dim
        self.c_q = nn.Linear(width, heads * head_dim, bias=False)
        self.c_k = nn.Linear(width, heads * head_dim, bias=False)
        self.c_v = nn.Linear(width, heads * head_dim, bias=False)
        self.c_proj = nn.Linear(heads * head_dim, width, bias=False)
        self.sq_proj = nn.Linear(width, heads * readout_dim, bias=False)
        self.sk_proj = nn.Linear(width, heads * readout_dim, bias=False)
        self.q_vocab = nn.Parameter(F.silu(torch.randn(heads, vocab_size, head_dim)))
        self.k_vocab = nn.Parameter(F.silu(torch.randn(heads, vocab_size, head_dim)))
        self.log_sel_tau = nn.Parameter(torch.empty(heads).uniform_(-4, 4))

    def forward(self, x, cos, sin, hard):
        from flash_dism import voc_dism
        b, n, _ = x.shape
        split = lambda t, d: t.view(b, n, self.heads, d)
        q, k, v = split(self.c_q(x), self.head_dim), split(self.c_k(x), self.head_dim), split(self.c_v(x), self.head_dim)
        q, k = rms(rotary(q, cos, sin)), rms(rotary(k, cos, sin))
        sq, sk = F.silu(split(self.sq_proj(x), self.readout_dim)), F.silu(split(self.sk_proj(x), self.readout_dim))
        tau = F.softplus(self.log_sel_tau.float())
        out = voc_dism(q, k, sq, sk, v, self.q_vocab, self.k_vocab, tau, direction=None, hard=hard)
        return self.c_proj(out.flatten(2))


class Block(nn.Module):
    def __init__(self, width, heads, head_dim):
        super().__init__()
        self.mixer = DismLayer(width, heads, head_dim)
        self.c_fc = nn.Linear(width, 4 * width, bias=False)
        self.c_out = nn.Linear(4 * width, width, bias=False)

    def forward(self, x, cos, sin, hard):
        x = x + self.mixer(rms(x), cos, sin, hard)
        return x + self.c_out(F.relu(self.c_fc(rms(x))).square())


class DismLM(nn.Module):
    """depth x (DISM layer + MLP); logits over `vocab` tokens; cross-entropy when targets are given."""

    def __init__(self, depth=20, width=1280, heads=10, head_dim=128, vocab=65536, rope_base=100000.):
        super().__init__()
        self.heads, self.head_dim, self.rope_base = heads, head_dim, rope_base
        self.embed = nn.Embedding(vocab, width)
        self.blocks = nn.ModuleList(Block(width, heads, head_dim) for _ in range(depth))
        self.unembed = nn.Linear(width, vocab, bias=False)

    def angles(self, n, device, dtype):
        inverse = 1. / self.rope_base ** (torch.arange(0, self.head_dim, 2, device=device, dtype=torch.float32) / self.head_dim)
        phase = torch.outer(torch.arange(n, device=device, dtype=torch.float32), inverse)
        return phase.cos()[:, None].to(dtype), phase.sin()[:, None].to(dtype)

    def forward(self, tokens, targets=None):
        b, n = tokens.shape
        x = rms(self.embed(tokens))
        cos, sin = self.angles(n, x.device, x.dtype)
        hard = torch.ones(b, self.heads, dtype=torch.bool, device=x.device)
        for block in self.blocks:
            x = block(x, cos, sin, hard)
        logits = self.unembed(rms(x))
        if targets is None:
            return logits
        return F.cross_entropy(logits.float().view(-1, logits.size(-1)), targets.reshape(-1))
