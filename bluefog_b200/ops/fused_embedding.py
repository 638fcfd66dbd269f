"""Token + position embedding of a GPT-style model on this library's kernels (``csrc/cuda/embed_kernels.cu``).

``token_position_embedding(idx, wte, wpe)`` is ``wte[idx] + wpe[arange(T)]`` for int64 ``idx`` [B, T] and bf16 CUDA
tables.  The backward pass adds the rows of repeated tokens in fp32 and returns dense gradients for both tables (the
position table's rows beyond T are zero).  Everything else - CPU, fp32 tables, deterministic algorithms requested -
takes PyTorch's embedding.  The reference has no model code of its own; this serves ``models/gpt2.py``.
"""
import os

import torch
import torch.nn.functional as F

from bluefog_b200.common.basics import get_basics

_b = get_basics()
ENABLED = os.environ.get("BLUEFOG_B200_EMBED", "1") != "0"       # 0: PyTorch's embedding everywhere
_INT_MAX = 2 ** 31 - 1
_scratch = {}        # (device, vocab, rows * C) -> (slot int32 [vocab] = INT_MAX, acc fp32 [rows * C] = 0)


def _eligible(idx, wte, wpe):
    C = _b.native
    return bool(ENABLED and C is not None and hasattr(C, "embed_forward") and idx.is_cuda and idx.dtype == torch.int64 and idx.dim() == 2
                and wte.is_cuda and wpe.is_cuda and wte.dtype == torch.bfloat16 and wpe.dtype == torch.bfloat16
                and wte.dim() == 2 and wpe.dim() == 2 and wte.shape[1] == wpe.shape[1] and wte.shape[1] % 8 == 0
                and idx.shape[1] <= wpe.shape[0] and idx.numel() > 0 and wte.is_contiguous() and wpe.is_contiguous()
                and not torch.are_deterministic_algorithms_enabled())


def _buffers(device, vocab, numel):
    key = (device, vocab, numel)
    buf = _scratch.get(key)
    if buf is None:
        buf = (torch.full((vocab,), _INT_MAX, dtype=torch.int32, device=device),
               torch.zeros(numel, dtype=torch.float32, device=device))
        _scratch[key] = buf
    return buf


class _EmbedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, wte, wpe):
        idx = idx.contiguous()
        out, bad = _b.native.embed_forward(idx, wte, wpe)
        ctx.save_for_backward(idx)
        ctx.tables = (wte.shape[0], wpe.shape[0])
        ctx.bad = bad           # set by the kernel when an index is outside the table; read by check_indices()
        _EmbedFn.last_bad = bad
        return out

    @staticmethod
    def backward(ctx, dx):
        (idx,) = ctx.saved_tensors
        vocab, positions = ctx.tables
        dx = dx.contiguous()
        slot, acc = _buffers(dx.device, vocab, dx.numel())
        d_wte, d_wpe = _b.native.embed_backward(idx, dx, vocab, slot, acc)
        if positions > d_wpe.shape[0]:
            d_wpe = F.pad(d_wpe, (0, 0, 0, positions - d_wpe.shape[0]))
        return None, d_wte, d_wpe


_EmbedFn.last_bad = None


def check_indices():
    """Raises IndexError if the last ``token_position_embedding`` call saw a token outside its table (the kernel skips
    such a token and sets a flag instead of faulting).  Synchronises with the device."""
    bad = _EmbedFn.last_bad
    if bad is not None and int(bad.item()) != 0:
        raise IndexError("token index out of range in token_position_embedding")


def token_position_embedding(idx, wte, wpe):
    """``wte[idx] + wpe[:T]`` with idx [B, T]."""
    if _eligible(idx, wte, wpe):
        return _EmbedFn.apply(idx, wte, wpe)
    t = idx.shape[1]
    return F.embedding(idx, wte) + wpe[:t]
