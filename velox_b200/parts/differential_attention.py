"""Differential attention over the paged KV cache.

Every head has two softmax maps over the same values; with a1 and a2 the maps' outputs

    o = a1 - lambda * a2;   o <- o / rms(o) * (1 - lambda_init);   o <- o * sigmoid(W_g x)

and ``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + lambda_init`` is one number of the layer.  The
projections hold both maps' rows head by head, [map 1, map 2] (``q.weight`` [H * 2 * dim, E],
``k.weight`` [G * 2 * dim, E]); ``v.weight`` [G * value_dim, E]; ``gate.weight`` and
``out.weight`` over H * value_dim.

How it runs on the engine's attention kernels: a cached key row of a KV head holds both maps'
keys side by side, [k map 1 | k map 2 | 0], ``head_dim`` wide; a query head becomes two rows,
[q map 1 | 0 | 0] and [0 | q map 2 | 0], whose products with the cached row are the two maps'
scores.  The kernels so see 2 H query heads over G KV heads of size ``head_dim`` and one set of
value pages, and both maps of a head share every K/V tile they read.  Before them, one kernel
norms (``qk_norm``: RMS over dim times ``q_norm`` / ``k_norm``, shared by heads and maps),
rotates (the position part's tables, on the first dims of every map) and places q, k and v;
after them, one kernel combines the maps, norms, scales and gates.  Options of the scores, all
parameters: ``softcap`` (``c tanh(s / c)``) and ``chunk`` (a query sees the keys of its own
chunk of positions, counted from 0); pages a chunk has left behind go back to the pool.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..ops import kernels
from ..ops.linear import linear, use_tensor_core_kernel
from .base import CacheNeeds, Mixer, PagedCacheSpec
from .registry import register_part


@register_part("mixer", "differential_attention")
class DifferentialAttention(Mixer):
    takes_padded_steps = True

    def __init__(self, params, weights, dtype, device, position=None) -> None:
        super().__init__(params, weights, dtype, device)
        self.hidden_size = E = int(params["hidden_size"])
        self.num_heads = H = int(params["num_heads"])
        self.num_kv_heads = G = int(params["num_kv_heads"])
        self.dim = dim = int(params["dim"])
        self.value_dim = vd = int(params["value_dim"])
        self.head_dim = D = int(params.get("head_dim") or -(-max(2 * dim, vd) // 16) * 16)
        self.softmax_scale = float(params["softmax_scale"])
        self.softcap = float(params.get("softcap") or 0.0)
        self.chunk = int(params.get("chunk") or 0)
        self.lambda_init = float(params["lambda_init"])
        self.eps = float(params["eps"])
        if H % G != 0:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if D % 16 != 0 or not 16 <= D <= 256 or 2 * dim > D or vd > D:
            raise ValueError(f"head_dim={D} must be a multiple of 16 up to 256 that holds 2 * dim={2 * dim} "
                             f"and value_dim={vd}")
        if position is None:
            raise ValueError("the differential attention mixer needs a position encoding part ('none' for none)")
        self.position = position
        self.rotary_dim = int(getattr(position, "rotary_dim", 0) or 0)
        if self.rotary_dim > dim:
            raise ValueError(f"rotary_dim={self.rotary_dim} exceeds dim={dim}")
        self.q_norm = self.k_norm = None
        if params.get("qk_norm", True):
            self.q_norm = self.expect("q_norm", (dim,))
            self.k_norm = self.expect("k_norm", (dim,))
        lam = [self.expect(name, (dim,)).to(torch.float32) for name in ("lq1", "lk1", "lq2", "lk2")]
        # One number of the layer, formed in float32 from the stored vectors.
        self.lam = float(torch.exp((lam[0] * lam[1]).sum()) - torch.exp((lam[2] * lam[3]).sum())) + self.lambda_init
        self.output_gate = bool(params.get("output_gate", True))
        self.q_width, self.k_width, self.v_width = 2 * H * dim, 2 * G * dim, G * vd
        self.gate_offset = self.q_width + self.k_width + self.v_width
        pieces = [self.expect("q.weight", (self.q_width, E)), self.expect("k.weight", (self.k_width, E)),
                  self.expect("v.weight", (self.v_width, E))]
        if self.output_gate:
            pieces.append(self.expect("gate.weight", (H * vd, E)))
        rows = sum(p.shape[0] for p in pieces)
        self.proj_width = -(-rows // 8) * 8
        if self.proj_width != rows:
            pieces.append(pieces[0].new_zeros(self.proj_width - rows, E))
        self.w_in = torch.cat(pieces).contiguous()
        self.w_out = self.expect("out.weight", (E, H * vd))
        for name in ("q.weight", "k.weight", "v.weight", "gate.weight"):
            self.weights.pop(name, None)
        self.rows_width = 2 * H * D
        kernels.heads()
        kernels.attention_lib(D)

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(paged=PagedCacheSpec(self.num_kv_heads, self.head_dim, None, chunk=self.chunk))

    def attention_signature(self):
        options = (("chunk", self.chunk),)
        return (self.num_kv_heads, 2 * self.num_heads // self.num_kv_heads, None, self.head_dim, 0, False, options)

    def forward(self, x, ctx, cache):
        T = ctx.num_tokens
        ws = ctx.workspace
        H, G, D = self.num_heads, self.num_kv_heads, self.head_dim
        if hasattr(x, "materialize"):
            x = x.materialize()
        proj = ws.get(f"differential.in{self.proj_width}", (ws.max_tokens, self.proj_width), self.dtype)
        linear(x, self.w_in, None, proj, T, status=ctx.status)
        group = ctx.groups[cache.group]
        k_cache, v_cache = (None, None) if cache.read_only else (cache.k, cache.v)
        # The rows the attention kernels read; what the placing kernel never writes stays zero,
        # so the buffer belongs to one (H, D, dim).
        rows = ws.get(f"differential.q{H}x{D}x{self.dim}", (ws.max_tokens, self.rows_width), self.dtype)
        cos = getattr(self.position, "cos", None) if self.rotary_dim else None
        sin = getattr(self.position, "sin", None) if self.rotary_dim else None
        kernels.diff_prepare(proj, rows, ctx.positions, cos, sin, self.q_norm, self.k_norm, self.eps,
                             group.slot_mapping, k_cache, v_cache, T, H, G, self.dim, self.value_dim, D,
                             self.rotary_dim, ctx.status)
        attn = ws.get(f"differential.maps{self.rows_width}", (ws.max_tokens, self.rows_width), self.dtype)
        plan = ctx.attention_plan(cache.group, self.attention_signature())
        for kind, items, count in plan.launches:
            kernels.attention(
                kind, rows, attn, cache.k, cache.v, group.block_tables, ctx.q_start, ctx.q_len, ctx.kv_len, items,
                count, plan.partial_o, plan.partial_lse, 2 * H, G, D, None, self.softmax_scale,
                merge_items=plan.merge_items, split_counters=plan.split_counters, status=ctx.status,
                cluster=plan.cluster if kind == kernels.ATTN_BF16_NARROW else 1,
                layout_checked=getattr(plan, "checked", False), softcap=self.softcap, chunk=self.chunk,
            )
        if hasattr(plan, "checked"):
            plan.checked = True
        if plan.num_merges and plan.split_counters is None:
            kernels.attention_merge(attn, ctx.q_start, plan.merge_items, plan.num_merges, plan.partial_o,
                                    plan.partial_lse, 2 * H, G, D, max_rows=plan.merge_rows)
        heads_out = ws.get(f"differential.out{H * self.value_dim}", (ws.max_tokens, H * self.value_dim), self.dtype)
        gate = proj[:, self.gate_offset : self.gate_offset + H * self.value_dim] if self.output_gate else None
        kernels.diff_combine(attn, gate, heads_out, T, H, self.value_dim, D, self.lam, 1.0 - self.lambda_init,
                             self.eps)
        if ctx.residual is not None and use_tensor_core_kernel(heads_out, self.w_out, T):
            # Few tokens: the projection is added straight into the float32 residual stream.
            linear(heads_out, self.w_out, None, ctx.residual, T, status=ctx.status, accumulate=True)
            return None
        out = ws.get("mixer.out", (ws.max_tokens, self.hidden_size), self.dtype)
        linear(heads_out, self.w_out, None, out, T, status=ctx.status)
        return out
