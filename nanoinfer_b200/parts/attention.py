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
                   StepLimits, StepPlan, Workspace, register_mixer)

#: a plan made for a graph rounds the longest key range of the decoded rows up to this many positions:
#: the split of the keys then stays the same from step to step while the requests grow
GRAPH_KEY_BUCKET = 256


class AttentionPlan(StepPlan):
    """Which rows of a step are single decoded tokens and which belong to prompt portions, and the
    portions cut into tiles of 64 and of 128 query rows, longest key range first; the same for
    every attention layer of the step.  Words: [decoded rows | portion rows (only beside decoded rows) |
    (entry, first row) per 64-row tile | the same per 128-row tile]."""

    def __init__(self, entry_start, entry_pos0, for_graph: bool = False, device=None):
        dec, pre, tiles = [], [], []
        self.max_decode_keys = 0
        #: for the trace's counts: keys seen by the decoded rows, keys seen by the portions' rows, and the
        #: key/value rows the portions' requests hold (each is read once)
        self.decode_keys = self.prefill_keys = self.prefill_kv_rows = 0
        for e in range(len(entry_start) - 1):
            a, b = entry_start[e], entry_start[e + 1]
            if b - a == 1:
                dec.append(a)
                self.max_decode_keys = max(self.max_decode_keys, entry_pos0[e] + 1)
                self.decode_keys += entry_pos0[e] + 1
            else:
                pre.extend(range(a, b))
                tiles.extend((e, off) for off in range(0, b - a, 64))
                n = b - a
                self.prefill_keys += n * entry_pos0[e] + n * (n + 1) // 2
                self.prefill_kv_rows += entry_pos0[e] + n
        # the same portions in tiles of 128 rows, for the tcgen05 kernel
        wide = [(e, off) for e in range(len(entry_start) - 1) if entry_start[e + 1] - entry_start[e] > 1
                for off in range(0, entry_start[e + 1] - entry_start[e], 128)]
        # the tiles that reach furthest back have the most keys to go through: they are launched first,
        # so that the short ones fill the gaps at the end
        tiles.sort(key=lambda t: -(entry_pos0[t[0]] + t[1]))
        wide.sort(key=lambda t: -(entry_pos0[t[0]] + t[1]))
        self.n_decode, self.n_prefill_rows, self.n_tiles = len(dec), len(pre), len(tiles)
        self.n_wide_tiles = len(wide)
        if for_graph:
            self.max_decode_keys = -(-self.max_decode_keys // GRAPH_KEY_BUCKET) * GRAPH_KEY_BUCKET
        # (the portions' rows are listed only beside decoded rows: alone they are the rows 0..n-1, and two
        # steps of portions that differ in a few tokens then have the same words' layout and one graph)
        self.n_listed_rows = len(pre) if dec else 0
        self.words = dec + (pre if dec else []) + [v for t in tiles for v in t] + [v for t in wide for v in t]
        if device is not None:
            self.bind(torch.tensor(self.words, dtype=torch.int32, device=device) if self.words else None)

    def graph_key(self) -> tuple:
        return (self.n_decode, self.n_listed_rows, self.n_tiles, self.n_wide_tiles, self.max_decode_keys)

    def bind(self, buf) -> None:
        """``buf``: a device int32 tensor holding ``self.words``."""
        nd, npre = self.n_decode, self.n_listed_rows
        all_decode = self.n_prefill_rows == 0
        # rows 0..n-1 in order need no index list
        self.decode_rows = None if all_decode or nd == 0 else buf[:nd]
        self.prefill_rows = None if nd == 0 or npre == 0 else buf[nd:nd + npre]
        self.tiles = buf[nd + npre:nd + npre + 2 * self.n_tiles] if self.n_tiles else None
        at = nd + npre + 2 * self.n_tiles
        self.wide_tiles = buf[at:at + 2 * self.n_wide_tiles] if self.n_wide_tiles else None


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

    def step_planner(self):
        return "causal_attention", AttentionPlan

    def flops_per_key(self) -> float:
        return 4.0 * self.q_dim

    def reserve(self, workspace: Workspace, limits: StepLimits) -> None:
        n = limits.max_rows
        workspace.reserve("attention.qkv", n * (self.q_dim + 2 * self.kv_dim), self.dtype)
        workspace.reserve("attention.out", n * self.q_dim, self.dtype)
        ops.attention_decode_reserve(workspace, self.n_head, self.head_dim)

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
            ops.trace_scope(ctx.layer, "qkv")
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
            ops.trace_scope(ctx.layer, "qkv")
            ops.linear(xn, p["qkv_weight"][:self.q_dim], None if qb is None else qb[:self.q_dim], q, T, norm=norm)
            if self.position is not None:
                self.position.on_qk(q[:T], None, ctx)
        att = ws.get("attention.out", (ctx.max_rows, self.q_dim), self.dtype)
        plan = ctx.plans.get("causal_attention")
        if plan is None:    # a caller that drives the part without the step function
            plan = ctx.plans["causal_attention"] = AttentionPlan(ctx.host_entry_start, ctx.host_entry_pos0,
                                                                 device=x.device)
        ops.attention(q, cache.layer, att, cache.block_table, ctx, self.n_head, self.scale, self.window, plan)
        ops.trace_scope(ctx.layer, "attn_proj")
        ops.linear(att, p["out_weight"], p.get("out_bias"), x, T, residual=True)
