"""GPT-2 (decoder-only transformer) with Hugging Face parameter names.

Used by the GPT-2-medium data-parallel workload (24 layers, d_model 1024, 16 heads, vocab
50257, sequence 1024).  The reference has no transformer code; the library only needs a
single-GPU model whose parameters the distributed optimizers average.  Linear layers run on
the hand-written tcgen05 GEMM when the activations are bf16 (``use_b200_gemm``), LayerNorm on the
row-in-registers kernels of ``bluefog_b200.ops.fused_ln``; attention uses PyTorch's fused
scaled-dot-product attention.
"""
import math

import os

import torch
import torch.nn as nn
import torch.nn.functional as F

from bluefog_b200.ops import fused_embedding
from bluefog_b200.ops.fused_ln import LayerNorm


class B200Linear(nn.Linear):
    """nn.Linear ([out, in] weight) that routes bf16 CUDA inputs to the tcgen05 GEMM."""

    def __init__(self, in_features, out_features, bias=True, use_b200_gemm=True, act=None):
        super().__init__(in_features, out_features, bias=bias)
        self.use_b200_gemm = use_b200_gemm

    def forward(self, x, residual=None):
        """``residual`` (same shape as the output) is added to the result; on the kernel path inside the GEMM epilogue."""
        if self.use_b200_gemm and x.is_cuda and x.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16:
            from bluefog_b200.ops import gemm
            if gemm.available() and self.in_features % 8 == 0:
                res2d = None if residual is None else residual.reshape(-1, self.out_features)
                y = gemm.linear(x.reshape(-1, self.in_features), self.weight, self.bias, res2d)
                return y.view(*x.shape[:-1], self.out_features)
        y = F.linear(x, self.weight, self.bias)
        return y if residual is None else y + residual


class Attention(nn.Module):
    def __init__(self, d_model, n_head, use_b200_gemm):
        super().__init__()
        self.n_head = n_head
        self.c_attn = B200Linear(d_model, 3 * d_model, use_b200_gemm=use_b200_gemm)
        self.c_proj = B200Linear(d_model, d_model, use_b200_gemm=use_b200_gemm)

    def forward(self, x, residual=None):
        b, t, c = x.shape
        q, k, v = self.c_attn(x).split(c, dim=2)
        shape = (b, t, self.n_head, c // self.n_head)
        q, k, v = (z.view(shape).transpose(1, 2) for z in (q, k, v))
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.c_proj(y.transpose(1, 2).reshape(b, t, c), residual)


class MLP(nn.Module):
    def __init__(self, d_model, use_b200_gemm):
        super().__init__()
        self.c_fc = B200Linear(d_model, 4 * d_model, use_b200_gemm=use_b200_gemm)
        self.c_proj = B200Linear(4 * d_model, d_model, use_b200_gemm=use_b200_gemm)

    def forward(self, x, residual=None):
        # BLUEFOG_B200_MLP_FUSION=0 keeps the GELU a kernel of its own between the two GEMMs
        if (self.c_fc.use_b200_gemm and x.is_cuda and x.dtype == torch.bfloat16
                and os.environ.get("BLUEFOG_B200_MLP_FUSION", "1") != "0"):
            from bluefog_b200.ops import gemm
            res2d = None if residual is None else residual.reshape(-1, residual.shape[-1])
            y = gemm.mlp_gelu(x.reshape(-1, x.shape[-1]), self.c_fc.weight, self.c_fc.bias, self.c_proj.weight,
                              self.c_proj.bias, res2d)
            return y.view(*x.shape[:-1], y.shape[-1])
        return self.c_proj(F.gelu(self.c_fc(x), approximate="tanh"), residual)


class Block(nn.Module):
    def __init__(self, d_model, n_head, use_b200_gemm):
        super().__init__()
        self.ln_1 = LayerNorm(d_model)
        self.attn = Attention(d_model, n_head, use_b200_gemm)
        self.ln_2 = LayerNorm(d_model)
        self.mlp = MLP(d_model, use_b200_gemm)

    def forward(self, x):
        # the residual stream joins each sub-layer's output inside the last GEMM's epilogue
        # and its two gradients (through the LayerNorm, and past it) meet inside the LayerNorm backward kernel
        h, x = self.ln_1.with_residual(x)
        x = self.attn(h, x)
        h, x = self.ln_2.with_residual(x)
        return self.mlp(h, x)


class GPT2(nn.Module):
    def __init__(self, vocab_size=50257, n_positions=1024, d_model=768, n_layer=12, n_head=12,
                 use_b200_gemm=True):
        super().__init__()
        self.wte = nn.Embedding(vocab_size, d_model)
        self.wpe = nn.Embedding(n_positions, d_model)
        self.h = nn.ModuleList([Block(d_model, n_head, use_b200_gemm) for _ in range(n_layer)])
        self.ln_f = LayerNorm(d_model)
        self.use_b200_gemm = use_b200_gemm
        self.apply(self._init)
        for name, p in self.named_parameters():
            if name.endswith("c_proj.weight"):
                nn.init.normal_(p, mean=0.0, std=0.02 / math.sqrt(2 * n_layer))

    @staticmethod
    def _init(m):
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, mean=0.0, std=0.02)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, mean=0.0, std=0.02)

    def forward(self, idx, targets=None):
        b, t = idx.shape
        x = fused_embedding.token_position_embedding(idx, self.wte.weight, self.wpe.weight)   # wte[idx] + wpe[:t]
        for block in self.h:
            x = block(x)
        x = self.ln_f(x)
        w = self.wte.weight                        # tied output embedding, [vocab, d_model]
        vocab = w.shape[0]
        pad = (-vocab) % 64 if x.is_cuda else 0
        if pad:
            # 50257 output columns make every GEMM of the classifier (forward, both gradients) run with
            # odd leading dimensions; the product is taken against the matrix padded to a multiple of
            # 64 rows and the surplus logits are set to -inf, which leaves loss and gradients unchanged
            w = F.pad(w, (0, 0, 0, pad))
        x2 = x.reshape(b * t, x.shape[-1])
        logits = None
        if self.use_b200_gemm and x2.is_cuda and x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
            from bluefog_b200.ops import gemm
            if gemm.available():
                logits = gemm.linear(x2, w)
        if logits is None:
            logits = F.linear(x2, w)
        if pad:
            logits[:, vocab:] = float("-inf")
        if targets is None:
            return logits[:, :vocab].reshape(b, t, vocab)
        from bluefog_b200.ops.fused_ce import cross_entropy
        return cross_entropy(logits, targets.reshape(-1))


def gpt2_small(**kw):
    return GPT2(d_model=768, n_layer=12, n_head=12, **kw)


def gpt2_medium(**kw):
    return GPT2(d_model=1024, n_layer=24, n_head=16, **kw)
