"""Attention over a cached low-rank latent.

Per token the layer caches one row: a latent ``c`` of ``kv_rank`` values (the first rows of the
down projection, RMS-normed) and one rotated key part of ``rot_dim`` values that all heads
share.  Head h's key is ``[W_uk[h] c | k_rot]`` and its value ``W_uv[h] c``; queries are laid out
head by head as ``[dim unrotated | rot_dim rotated]``.  Because the unrotated score
``q_u . (W_uk[h] c)`` equals ``(W_uk[h]^T q_u) . c``, the step never expands keys or values:

    proj  = [side rows ; W_q ; W_dkv ; W_g] x            one projection of the layer's input
    c, k_rot -> cache;  q_rot rotated                    kernels.latent_prepare
    q_abs[h] = W_uk[h]^T q_u[h]                          kernels.headwise_linear
    o_lat[h] = softmax(([q_abs[h] | q_rot[h]] . [c | k_rot]) * scale) applied to the rows c
                                                         the paged attention kernels, one shared
                                                         KV head whose rows are keys and values
    o[h]     = sigmoid(g[h]) * W_uv[h] o_lat[h]          kernels.headwise_linear with the gate
    out      = W_o o

A layer with ``own_latent`` false has no down projection: it reads the cache of the schedule entry
named by the model's schedule (``cache.read_only``) with its own W_uk, W_uv and queries.

``side_rows`` > 0: the first rows of ``in.weight`` are not the mixer's; their products (plus
``side.bias``) belong to the block around it and are handed over as ``ctx.side_output``.

Further forms, all chosen by parameters.  ``query_rank`` r > 0: the queries come through a latent
of their own, ``q = W_uq rms_norm(W_dq x) * w``; ``in.weight`` then holds the r rows of W_dq where
it otherwise holds W_q, and the part has ``uq.weight`` and ``query_norm.weight``.  ``window``: a
query sees itself and the ``window - 1`` keys before it.  ``sink``: a learned number per head
whose exponential joins the softmax denominator (weight ``sink``).  ``gate`` "element": the gate
is ``sigmoid(W_g x)`` over all ``heads * value_dim`` outputs, not one number per head.  The
position part decides which dims are a rotating pair (``layout``: neighbours, or dim i with dim
i + pairs).

A cached row of ``kv_rank + rot_dim`` values must fit the attention kernels' widest row (256).  A
wider latent (with ``query_rank``) runs in the expanded form instead (``form``: "absorbed",
"expanded", or "auto", which picks by that width): keys ``[k_rot | W_uk[h] c]`` and values
``W_uv[h] c`` are made per head by one projection of ``[normed query latent | k_rot | c]`` whose
matrix holds W_uq, W_uk, W_uv and an identity for the shared part (rotated dims first in every
head, so the engine's rotate-and-store kernel takes them), cached per head, and attended to as
ordinary heads; the pages then cost ``2 * heads * head_dim`` values a token instead of one row.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import linear
from .base import CacheNeeds, Mixer, PagedCacheSpec
from .registry import register_part


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    takes_padded_steps = True

    def __init__(self, params, weights, dtype, device, position=None) -> None:
        super().__init__(params, weights, dtype, device)
        self.hidden_size = int(params["hidden_size"])
        self.num_heads = int(params["num_heads"])
        self.dim = int(params["dim"])
        self.rot_dim = int(params["rot_dim"])
        self.value_dim = int(params["value_dim"])
        self.kv_rank = int(params["kv_rank"])
        self.softmax_scale = float(params["softmax_scale"])
        self.eps = float(params["eps"])
        self.own_latent = bool(params.get("own_latent", True))
        self.gated = bool(params.get("output_gate", True))
        self.gate_each = params.get("gate", "head") == "element"
        if params.get("gate", "head") not in ("head", "element"):
            raise ValueError(f"latent attention: gate is 'head' or 'element', not {params.get('gate')!r}")
        self.side_rows = int(params.get("side_rows", 0))
        self.query_rank = int(params.get("query_rank") or 0)
        self.window = params.get("window")
        if position is None or not hasattr(position, "pairs"):
            raise ValueError("latent attention needs a pair-rotating position encoding part")
        self.half_layout = getattr(position, "layout", "pairs") == "half"
        if 2 * position.pairs > self.rot_dim:
            raise ValueError(f"the rotation covers {2 * position.pairs} dims, the rotated part has {self.rot_dim}")
        self.position = position
        # A cached row, padded to what the attention kernels take (a multiple of 16 up to 256).
        self.row_dim = -(-(self.kv_rank + self.rot_dim) // 16) * 16
        form = params.get("form", "auto")
        if form not in ("auto", "absorbed", "expanded"):
            raise ValueError(f"latent attention: form is 'auto', 'absorbed' or 'expanded', not {form!r}")
        self.expanded = form == "expanded" or (form == "auto" and self.row_dim > 256 and self.query_rank > 0)
        if self.row_dim > 256 and not self.expanded:
            raise ValueError(
                f"kv_rank + rot_dim = {self.kv_rank + self.rot_dim} is more than the attention kernels' "
                "largest row of 256 (the expanded form takes wider latents of layers with a query latent)"
            )
        H, q_head = self.num_heads, self.dim + self.rot_dim
        self.q_offset = self.side_rows
        self.latent_offset = self.q_offset + (self.query_rank if self.query_rank else H * q_head)
        self.gate_offset = self.latent_offset + (self.kv_rank + self.rot_dim if self.own_latent else 0)
        self.gate_rows = (H * self.value_dim if self.gate_each else H) if self.gated else 0
        rows = self.gate_offset + self.gate_rows
        self.w_in = self.expect("in.weight", (rows, self.hidden_size))
        # Rows of zeros up to a multiple of eight: the projection's output rows then start on
        # 16-byte boundaries in bfloat16, which the library GEMM of long steps and the vector
        # loads of the kernels that read the columns want.
        self.in_width = -(-rows // 8) * 8
        if self.in_width != rows:
            self.w_in = torch.cat([self.w_in, self.w_in.new_zeros(self.in_width - rows, self.hidden_size)]).contiguous()
        self.b_in = None
        self.b_in_lowp = None
        if self.side_rows and "side.bias" in weights:
            side = self.expect("side.bias", (self.side_rows,))
            self.b_in = torch.cat([side, side.new_zeros(self.in_width - self.side_rows)]).contiguous()
            if dtype != torch.float32:
                self.b_in_lowp = self.b_in.to(dtype)
        self.latent_norm = self.expect("latent_norm.weight", (self.kv_rank,)) if self.own_latent else None
        self.w_uq = self.query_norm = None
        if self.query_rank:
            # The normed query latent is padded with zeros to whole 16-byte rows; the matching
            # columns of W_uq are zero.
            self.query_norm = self.expect("query_norm.weight", (self.query_rank,))
            w_uq = self.expect("uq.weight", (H * q_head, self.query_rank))
            self.query_rank_padded = -(-self.query_rank // 8) * 8
            if self.query_rank_padded != self.query_rank:
                w_uq = torch.cat([w_uq, w_uq.new_zeros(H * q_head, self.query_rank_padded - self.query_rank)], dim=1)
            self.w_uq = w_uq.contiguous()
        self.sink = self.expect("sink", (H,)) if params.get("sink", False) else None
        # W_uk [H * dim, kv_rank] is used transposed per head (the contraction runs over dim).
        w_uk = self.expect("uk.weight", (H * self.dim, self.kv_rank))
        self.w_uk_t = w_uk.view(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = self.expect("uv.weight", (H * self.value_dim, self.kv_rank)).view(H, self.value_dim, self.kv_rank)
        self.w_out = self.expect("out.weight", (self.hidden_size, H * self.value_dim))
        if self.expanded:
            self._build_expanded(w_uk)
        kernels.attention_lib(self.head_dim if self.expanded else self.row_dim)

    def _build_expanded(self, w_uk: torch.Tensor) -> None:
        """The one matrix of the expanded form.  Its input columns are ``[normed query latent (padded) |
        k_rot | c (padded)]``; its rows are, head by head, the queries ``[rotated | unrotated | 0]``,
        then the keys ``[k_rot | W_uk[h] c | 0]`` (an identity copies the shared part into every head),
        then the values ``[W_uv[h] c | 0]``, every head ``head_dim`` rows."""
        if not (self.query_rank and self.own_latent and not self.side_rows):
            raise ValueError("the expanded form of latent attention needs a query latent, a down projection of "
                             "its own and no side rows")
        H, D, R, V, rank = self.num_heads, self.dim, self.rot_dim, self.value_dim, self.kv_rank
        self.head_dim = Dh = -(-max(D + R, V) // 16) * 16
        if Dh > 256:
            raise ValueError(f"heads of {max(D + R, V)} values are more than the attention kernels' largest of 256")
        Cq = self.query_rank_padded
        cols = -(-(Cq + R + rank) // 8) * 8
        self.x_cols, self.x_rot_at, self.x_latent_at = cols, Cq, Cq + R
        w_uq = self.w_uq.view(H, D + R, Cq)
        big = w_uq.new_zeros(3 * H, Dh, cols)
        big[:H, :R, :Cq] = w_uq[:, D:]
        big[:H, R : R + D, :Cq] = w_uq[:, :D]
        big[H : 2 * H, :R, Cq : Cq + R] = torch.eye(R, dtype=big.dtype, device=big.device)
        big[H : 2 * H, R : R + D, Cq + R : Cq + R + rank] = w_uk.view(H, D, rank)
        big[2 * H :, :V, Cq + R : Cq + R + rank] = self.w_uv
        self.w_heads = big.reshape(3 * H * Dh, cols).contiguous()
        # The heads' first ``value_dim`` values, gated: a per-head product with an identity.
        pick = w_uq.new_zeros(H, V, Dh)
        pick[:, :, :V] = torch.eye(V, dtype=pick.dtype, device=pick.device)
        self.w_pick = pick.contiguous()
        kernels.mixers()

    def cache_needs(self) -> CacheNeeds:
        if self.expanded:
            return CacheNeeds(paged=PagedCacheSpec(self.num_heads, self.head_dim, self.window))
        return CacheNeeds(paged=PagedCacheSpec(1, self.row_dim, self.window, values_in_keys=True))

    def attention_signature(self):
        base = ((self.num_heads, 1, self.window, self.head_dim) if self.expanded
                else (1, self.num_heads, self.window, self.row_dim))
        # A sink comes in where split key ranges are merged: such rows always take that way.
        return base + (0, True) if self.sink is not None else base

    def _attend(self, queries, attn, cache, ctx, kv_heads, head_dim):
        group = ctx.groups[cache.group]
        H = self.num_heads
        plan = ctx.attention_plan(cache.group, self.attention_signature())
        for kind, items, count in plan.launches:
            kernels.attention(
                kind, queries, attn, cache.k, cache.v, group.block_tables, ctx.q_start, ctx.q_len,
                ctx.kv_len, items, count, plan.partial_o, plan.partial_lse, H, kv_heads, head_dim, self.window,
                self.softmax_scale, merge_items=plan.merge_items, split_counters=plan.split_counters,
                status=ctx.status,
                cluster=(plan.cluster if kind == kernels.ATTN_BF16_NARROW else
                         getattr(plan, "tc_ctas_per_sm", 1) if kind == kernels.ATTN_BF16_TC else 1),
                layout_checked=getattr(plan, "checked", False),
            )
        if hasattr(plan, "checked"):
            plan.checked = True
        if plan.num_merges and plan.split_counters is None:
            kernels.attention_merge(
                attn, ctx.q_start, plan.merge_items, plan.num_merges, plan.partial_o, plan.partial_lse,
                H, kv_heads, head_dim, max_rows=plan.merge_rows, sinks=self.sink,
            )

    def _forward_expanded(self, x, ctx, cache):
        T = ctx.num_tokens
        ws = ctx.workspace
        H, Dh, R, rank = self.num_heads, self.head_dim, self.rot_dim, self.kv_rank
        proj = ws.get(f"latent.proj{self.in_width}", (ws.max_tokens, self.in_width), self.dtype)
        linear(x, self.w_in, None, proj, T, status=ctx.status)
        # [normed query latent | k_rot | normed latent], each norm filling its padding with zeros.
        both = ws.get(f"latent.both{self.x_cols}", (ws.max_tokens, self.x_cols), self.dtype)
        kernels.rms_rows(proj[:, self.q_offset : self.q_offset + self.query_rank], self.query_norm, self.eps,
                         both[:, : self.x_rot_at], T)
        at = self.latent_offset
        kernels.act_rows(proj[:, at + rank : at + rank + R], both[:, self.x_rot_at : self.x_latent_at], T,
                         kernels.ACT_NONE)
        kernels.rms_rows(proj[:, at : at + rank], self.latent_norm, self.eps, both[:, self.x_latent_at :], T)
        qkv = ws.get(f"latent.heads_qkv{3 * H * Dh}", (ws.max_tokens, 3 * H * Dh), self.dtype)
        linear(both, self.w_heads, None, qkv, T, status=ctx.status)
        group = ctx.groups[cache.group]
        rotating = 2 * self.position.pairs
        if self.half_layout:
            kernels.rope_cache_write(qkv, ctx.positions, self.position.cos, self.position.sin, group.slot_mapping,
                                     cache.k, cache.v, T, H, H, Dh, rotating, ctx.status)
        else:
            kernels.pair_rope_cache_write(qkv, ctx.positions, self.position.cos, self.position.sin, group.slot_mapping,
                                          cache.k, cache.v, T, H, H, Dh, rotating, ctx.status)
        attn = ws.get(f"latent.attn{H * Dh}", (ws.max_tokens, H * Dh), self.dtype)
        self._attend(qkv, attn, cache, ctx, H, Dh)
        heads_out = ws.get(f"latent.heads{H * self.value_dim}", (ws.max_tokens, H * self.value_dim), self.dtype)
        kernels.headwise_linear(attn, 0, Dh, self.w_pick, heads_out, 0, self.value_dim, T,
                                gate=proj if self.gated else None, gate_offset=self.gate_offset,
                                gate_each=self.gate_each)
        out = ws.get("mixer.out", (ws.max_tokens, self.hidden_size), self.dtype)
        linear(heads_out, self.w_out, None, out, T, status=ctx.status)
        return out

    def forward(self, x, ctx, cache):
        if self.expanded:
            return self._forward_expanded(x, ctx, cache)
        T = ctx.num_tokens
        ws = ctx.workspace
        H, Dp = self.num_heads, self.row_dim
        if cache.read_only == self.own_latent:
            raise ValueError("a latent-attention layer writes the cache exactly when it has a down projection")
        # Buffers are named by their width: layers of different sizes must not take turns
        # reallocating one name (a captured step keeps the addresses it was captured with).
        proj = ws.get(f"latent.proj{self.in_width}", (ws.max_tokens, self.in_width), self.dtype)
        linear(x, self.w_in, self.b_in, proj, T, self.b_in_lowp, status=ctx.status)
        ctx.side_output = proj[:, : self.side_rows] if self.side_rows else None

        queries = ws.get(f"latent.queries{H * Dp}", (ws.max_tokens, H * Dp), self.dtype)
        group = ctx.groups[cache.group]
        q_rows, q_offset = proj, self.q_offset
        if self.query_rank:
            # The queries' own latent: norm, then the second projection.
            q_width = H * (self.dim + self.rot_dim)
            latent_q = ws.get(f"latent.query_latent{self.query_rank_padded}", (ws.max_tokens, self.query_rank_padded),
                              self.dtype)
            kernels.rms_rows(proj[:, self.q_offset : self.q_offset + self.query_rank], self.query_norm, self.eps,
                             latent_q, T)
            q_rows, q_offset = ws.get(f"latent.q{q_width}", (ws.max_tokens, q_width), self.dtype), 0
            linear(latent_q, self.w_uq, None, q_rows, T, status=ctx.status)
        kernels.latent_prepare(
            proj, q_offset, self.latent_offset if self.own_latent else None, ctx.positions, self.position.cos,
            self.position.sin, self.latent_norm, self.eps, group.slot_mapping, cache.k,
            queries.view(ws.max_tokens, H, Dp), T, H, self.dim, self.rot_dim, self.kv_rank, ctx.status,
            half_layout=self.half_layout, q_source=q_rows if self.query_rank else None,
        )
        kernels.headwise_linear(q_rows, q_offset, self.dim + self.rot_dim, self.w_uk_t, queries, 0, Dp, T)

        attn = ws.get(f"latent.attn{H * Dp}", (ws.max_tokens, H * Dp), self.dtype)
        self._attend(queries, attn, cache, ctx, 1, Dp)

        heads_out = ws.get(f"latent.heads{H * self.value_dim}", (ws.max_tokens, H * self.value_dim), self.dtype)
        kernels.headwise_linear(attn, 0, Dp, self.w_uv, heads_out, 0, self.value_dim, T,
                                gate=proj if self.gated else None, gate_offset=self.gate_offset,
                                gate_each=self.gate_each)
        out = ws.get("mixer.out", (ws.max_tokens, self.hidden_size), self.dtype)
        linear(heads_out, self.w_out, None, out, T, status=ctx.status)
        return out
