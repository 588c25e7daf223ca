"""Causal multi-head attention over the paged cache, with a fused query/key/value projection
and an output projection whose epilogue adds into the residual stream.

Reference: qkv = ln_1(x) . W^T + b with the row laid out [q | k | v] and head h owning
columns h*hd..(h+1)*hd of each third (crates/core/src/stages/blocks.rs:31-50); keys and values
appended to the cache after the bias (crates/core/src/stages/kv_cache.rs:44-57); scores
(q . k) * scale over the keys j <= pos, softmax, weighted sum of values
(crates/core/src/kernels/reference.rs:109-142); x += att . W_proj^T + b (blocks.rs:103-112).
The reference fixes scale = 1/sqrt(hd) and one key/value head per query head; here the
scale, the number of key/value heads, the head size and a window are parameters.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import ops
from .base import (MATRIX, VECTOR, KVCacheSpec, KVCacheView, Mixer, ParamSpec, PositionEncoding, StepContext,
                   register_mixer)


def _split(xn):
    """(tensor, norm input): a part's input is either the normed rows or a foldable norm input."""
    return (None, xn) if isinstance(xn, ops.NormInput) else (xn, None)


@register_mixer("causal_attention")
class CausalSelfAttention(Mixer):
    takes_norm_input = True

    def __init__(self, width: int, n_head: int, n_kv_head: int, head_dim: int, scale: float,
                 window: int = 0, bias: bool = True, position: Optional[PositionEncoding] = None):
        if n_head <= 0 or n_kv_head <= 0 or n_head % n_kv_head != 0:
            raise ValueError(f"n_head {n_head} must be a positive multiple of n_kv_head {n_kv_head}")
        if head_dim <= 0 or head_dim % 8 != 0 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim} is not supported: it must be a multiple of 8, at most 256")
        if window < 0:
            raise ValueError("window must be >= 0")
        self.width, self.n_head, self.n_kv_head, self.head_dim = int(width), int(n_head), int(n_kv_head), int(head_dim)
        self.scale, self.window, self.bias, self.position = float(scale), int(window), bool(bias), position
        self.q_dim = self.n_head * self.head_dim
        self.kv_dim = self.n_kv_head * self.head_dim

    def param_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec("qkv_weight", (self.q_dim + 2 * self.kv_dim, self.width), MATRIX),
                 ParamSpec("out_weight", (self.width, self.q_dim), MATRIX)]
        if self.bias:
            specs += [ParamSpec("qkv_bias", (self.q_dim + 2 * self.kv_dim,), VECTOR),
                      ParamSpec("out_bias", (self.width,), VECTOR)]
        return specs

    def kv_spec(self) -> Optional[KVCacheSpec]:
        return KVCacheSpec(self.n_kv_head, self.head_dim, self.window)

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: Optional[KVCacheView],
                state: Optional[torch.Tensor], writes_cache: bool = True) -> None:
        if cache is None:
            raise ValueError("causal_attention needs a paged cache")
        T, p = ctx.n_rows, self.params
        ws = ctx.workspace
        xn, norm = _split(xn)
        if writes_cache:
            qkv = ws.get("attention.qkv", (ctx.max_rows, self.q_dim + 2 * self.kv_dim), self.dtype)
            # small steps: keys and values go to the cache from the projection's epilogue
            fused = self.position is None and ops.linear_qkv(
                xn, p["qkv_weight"], p.get("qkv_bias"), qkv, T, self.q_dim, cache.layer, cache.block_table,
                ctx.row_entry, ctx.positions, ctx.status, norm=norm)
            if not fused:
                ops.linear(xn, p["qkv_weight"], p.get("qkv_bias"), qkv, T, norm=norm)
                if self.position is not None:
                    self.position.on_qk(qkv[:T, :self.q_dim], qkv[:T, self.q_dim:self.q_dim + self.kv_dim], ctx)
                ops.kv_append(qkv, self.q_dim, self.q_dim + self.kv_dim, cache.layer, cache.block_table,
                              ctx.row_entry, ctx.positions, T, ctx.status)
            q = qkv[:, :self.q_dim]
        else:
            # this layer reads another layer's keys and values: only the queries are projected
            q = ws.get("attention.q", (ctx.max_rows, self.q_dim), self.dtype)
            qb = p.get("qkv_bias")
            ops.linear(xn, p["qkv_weight"][:self.q_dim], None if qb is None else qb[:self.q_dim], q, T, norm=norm)
            if self.position is not None:
                self.position.on_qk(q[:T], None, ctx)
        att = ws.get("attention.out", (ctx.max_rows, self.q_dim), self.dtype)
        ops.attention(q, cache.layer, att, cache.block_table, ctx, self.n_head, self.scale, self.window)
        ops.linear(att, p["out_weight"], p.get("out_bias"), x, T, residual=True)
