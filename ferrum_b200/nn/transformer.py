"""Attention and transformer pieces (ferrum-nn/src/transformer.rs:10-403).

``MultiHeadAttention`` projects with Linear layers (GEMM kernels; 3-D inputs work, unlike the reference where the
3-D matmul is unimplemented), computes ``softmax(Q K^T / sqrt(d)) V`` per head with the batched GEMM and the row
softmax kernel, and is differentiable.  Under autocast both products run on the batched tcgen05 kernel directly
on the head-interleaved ``[B, S, H, D]`` projections (4-D TMA maps; no head-split or transpose copies), with the
1/sqrt(d) scale in the first product's epilogue and the second product written back in ``[B, S, H, D]`` order.  ``TransformerEncoderLayer`` is post-LayerNorm with a ReLU feed-forward, as
in the reference; ``PositionalEncoding`` is the fixed sinusoid table.
"""
from __future__ import annotations

import math

import torch

from .. import config
from ..core import ShapeMismatch, _as_device
from ..ops import functional as F
from .modules import LayerNorm, Linear, Module, tensor_io


class MultiHeadAttention(Module):
    """Under autocast with head dimension 64 or 128 and no explicit mask (``causal=True`` is fine) the attention core
    runs on the blockwise tcgen05 kernels in both directions: no S x S matrix is stored for the backward pass, the
    probabilities are recomputed tile by tile from one log-sum-exp per row.  Other head dimensions, explicit
    masks and fp32 precision take the batched-GEMM + softmax path (``memory_efficient=True`` then recomputes the
    scores in the backward pass where the blockwise forward applies)."""

    def __init__(self, embed_dim: int, num_heads: int, device=None, memory_efficient: bool = False):
        super().__init__()
        self.memory_efficient = bool(memory_efficient)
        if embed_dim % num_heads:
            raise ValueError("embed_dim must be divisible by num_heads")
        self.embed_dim, self.num_heads, self.head_dim = int(embed_dim), int(num_heads), embed_dim // num_heads
        self.q_proj = Linear(embed_dim, embed_dim, device=device)
        self.k_proj = Linear(embed_dim, embed_dim, device=device)
        self.v_proj = Linear(embed_dim, embed_dim, device=device)
        self.out_proj = Linear(embed_dim, embed_dim, device=device)

    @classmethod
    def new(cls, embed_dim, num_heads):
        return cls(embed_dim, num_heads)

    def _split(self, t, B, S):
        return t.reshape(B, S, self.num_heads, self.head_dim).transpose(1, 2)  # [B, H, S, D]

    @tensor_io
    def forward_attn(self, query, key, value, mask=None, causal: bool = False):
        if query.dim() != 3 or query.shape[-1] != self.embed_dim:
            raise ShapeMismatch("MultiHeadAttention", f"[B, S, {self.embed_dim}]", list(query.shape))
        B, Sq, _ = query.shape
        Sk = key.shape[1]
        q = self._split(self.q_proj(query), B, Sq)
        k = self._split(self.k_proj(key), B, Sk)
        v = self._split(self.v_proj(value), B, Sk)
        if causal and Sk < Sq:
            raise ShapeMismatch("MultiHeadAttention(causal)", "at least as many keys as queries", [Sq, Sk])
        if (mask is None and self.head_dim in (64, 128) and config.low_precision_active()
                and F.flash_attention_ok(q, k, v)):
            # inference (no gradient needed), bf16: blockwise attention, the score matrix is never materialised
            ctx = F.flash_attention(q, k, v, 1.0 / math.sqrt(self.head_dim), causal=causal)
            return self.out_proj(ctx.transpose(1, 2).reshape(B, Sq, self.embed_dim))
        if (mask is None and self.head_dim in (64, 128) and config.low_precision_active()
                and F.flash_attention_ok(q, k, v, need_no_grad=False)):
            # training, bf16: blockwise forward AND backward, nothing of size S x S in memory
            ctx = F.attention_blockwise(q, k, v, 1.0 / math.sqrt(self.head_dim), causal=causal)
            return self.out_proj(ctx.transpose(1, 2).reshape(B, Sq, self.embed_dim))
        if causal:  # the differentiable paths take the causal structure as an additive mask
            i = torch.arange(Sq, device=q.device)[:, None]
            j = torch.arange(Sk, device=q.device)[None, :]
            cm = j <= i + (Sk - Sq)
            mask = cm if mask is None else (mask & cm if mask.dtype == torch.bool else mask.masked_fill(~cm, -1e9))
        if (self.memory_efficient and mask is None and self.head_dim in (64, 128) and config.low_precision_active()
                and F.flash_attention_ok(q, k, v, need_no_grad=False)):
            # training without S x S activations: blockwise forward, scores recomputed in the backward pass
            ctx = F.attention_checkpointed(q, k, v, 1.0 / math.sqrt(self.head_dim))
            return self.out_proj(ctx.transpose(1, 2).reshape(B, Sq, self.embed_dim))
        scores = F.bmm_scaled(q, k.transpose(-1, -2), 1.0 / math.sqrt(self.head_dim))  # scale in the GEMM epilogue
        if mask is not None:
            m = mask.to(scores.dtype) if mask.dtype != torch.bool else torch.zeros_like(
                mask, dtype=scores.dtype).masked_fill(~mask, -1e9)
            scores = F.binary(scores, m, "add")
        attn = F.softmax(scores, -1)
        ctx = F.bmm_scaled(attn, v, 1.0, heads_inner=True)            # [B, H, Sq, D], stored [B, Sq, H, D]
        ctx = ctx.transpose(1, 2).reshape(B, Sq, self.embed_dim)
        return self.out_proj(ctx)

    def forward(self, x):
        return self.forward_attn(x, x, x)


class TransformerEncoderLayer(Module):
    def __init__(self, d_model: int, nhead: int, dim_feedforward: int, device=None):
        super().__init__()
        self.self_attn = MultiHeadAttention(d_model, nhead, device=device)
        self.linear1 = Linear(d_model, dim_feedforward, device=device)
        self.linear2 = Linear(dim_feedforward, d_model, device=device)
        self.norm1 = LayerNorm([d_model], device=device)
        self.norm2 = LayerNorm([d_model], device=device)

    @classmethod
    def new(cls, d_model, nhead, dim_feedforward):
        return cls(d_model, nhead, dim_feedforward)

    @tensor_io
    def forward(self, x):
        x = self.norm1(F.binary(x, self.self_attn(x), "add"))
        ff = self.linear2(self.linear1._forward_act(x, "relu") if x.is_cuda else F.unary(self.linear1(x), "relu"))
        return self.norm2(F.binary(x, ff, "add"))


class PositionalEncoding(Module):
    def __init__(self, d_model: int, max_len: int = 5000, device=None):
        super().__init__()
        pos = torch.arange(max_len, dtype=torch.float32).unsqueeze(1)
        div = torch.exp(torch.arange(0, d_model, 2, dtype=torch.float32) * (-math.log(10000.0) / d_model))
        pe = torch.zeros(max_len, d_model)
        pe[:, 0::2] = torch.sin(pos * div)
        pe[:, 1::2] = torch.cos(pos * div)[:, : d_model // 2]
        self.register_buffer("pe", pe.to(_as_device(device).to_torch()))
        self.d_model, self.max_len = d_model, max_len

    @classmethod
    def new(cls, d_model, max_len):
        return cls(d_model, max_len)

    @tensor_io
    def forward(self, x):
        S = x.shape[-2]
        if S > self.max_len:
            raise ShapeMismatch("PositionalEncoding", f"sequence <= {self.max_len}", S)
        return F.binary(x, self.pe[:S].to(x.dtype), "add")
