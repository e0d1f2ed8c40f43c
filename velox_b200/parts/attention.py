"""Attention mixer over the paged KV cache.

One forward is: fused q/k/v projection (+bias) -> position encoding on q and k, k and v written
to the cache -> attention of the step's rows over the cache -> output projection
(src/self_attention.py:48-90 of the reference).  A step's tokens attend to themselves through
the cache: the write comes first.  Whether a row belongs to a prompt portion or is a single
decoded token makes no difference here; the step's work layout decides which kernel family
runs which rows.

Optional forms, all chosen by parameters: heads whose query/key size and value size differ and
need not be multiples of 16 (``key_dim``, ``value_dim``: the projections are laid out with every
head padded with zeros to ``head_dim``, which is what the kernels see); a window that keeps the
first ``keep_first`` keys; a learned sink per head in the softmax denominator (``sink``); a gate
per head on the heads' outputs, ``sigmoid(W_g x)`` (``head_gate``: its rows ride along behind
q | k | v in the one projection); ``values_from_keys``: there is no value projection, a token's
values are its keys as projected (bias included), before the rotation.  Such a part takes its
matrices as ``q.weight``, ``k.weight``, ``v.weight`` (and biases) instead of one ``qkv.weight``.

Changes to the scores, made inside the attention kernels: ``distance_bias`` (weights ``bias_r1``,
``bias_r2``, one number each per query head): ``r1 ln(1 + r2 (i - j))`` is taken off the score of
query i and key j; ``sink_zero``: one more term of score 0 and no value in every softmax
denominator (without a window); a position part with a ``row_scale`` table (``log_temperature``)
multiplies a query's scores by a number that depends on its position.  Every kernel family takes
them.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..ops import kernels
from ..ops.linear import linear, qkv_rope_linear, use_tensor_core_kernel
from .base import CacheNeeds, Mixer, PagedCacheSpec
from .registry import register_part

# VELOX_B200_NO_ROPE_FUSION=1 always rotates in a kernel of its own (for bisecting).
_FUSE_ROPE = os.environ.get("VELOX_B200_NO_ROPE_FUSION") != "1"


@register_part("mixer", "attention")
class Attention(Mixer):
    def __init__(self, params, weights, dtype, device, position=None) -> None:
        super().__init__(params, weights, dtype, device)
        self.hidden_size = int(params["hidden_size"])
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.window: Optional[int] = params.get("window")
        self.softmax_scale = float(params["softmax_scale"])
        if self.num_heads % self.num_kv_heads != 0:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.head_dim % 16 != 0 or not 16 <= self.head_dim <= 256:
            raise ValueError(
                f"head_dim={self.head_dim} is not supported by the attention kernels "
                "(a multiple of 16 between 16 and 256)"
            )
        if position is None:
            raise ValueError("the attention mixer needs a position encoding part ('none' for none)")
        self.position = position
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        self.qkv_width = self.q_size + 2 * self.kv_size
        self.keep_first = int(params.get("keep_first") or 0) if self.window else 0
        self.sink = self.expect("sink", (self.num_heads,)) if params.get("sink", False) else None
        # Rows finished by the merge kernel: that is where a sink and the kept first keys come in.
        self.anchored = self.sink is not None or self.keep_first > 0
        self.head_gate = bool(params.get("head_gate", False))
        self.sink_zero = bool(params.get("sink_zero", False))
        if self.sink_zero and (self.window or self.sink is not None):
            raise ValueError("attention: sink_zero goes with neither a window nor a learned sink")
        self.distance_bias = None
        if params.get("distance_bias", False):
            self.distance_bias = (self.expect("bias_r1", (self.num_heads,)), self.expect("bias_r2", (self.num_heads,)))
        self.row_scale = getattr(position, "row_scale", None)
        self.b_qkv = None
        self.b_qkv_lowp = None
        self.values_from_keys = False
        if "qkv.weight" in weights:
            self.proj_width = self.qkv_width
            self.w_qkv = self.expect("qkv.weight", (self.qkv_width, self.hidden_size))
            if params.get("qkv_bias", False):
                self.b_qkv = self.expect("qkv.bias", (self.qkv_width,))
            self.w_out = self.expect("out.weight", (self.hidden_size, self.q_size))
        else:
            self._fuse_padded(params, dtype, device)
        if self.b_qkv is not None and dtype != torch.float32:
            self.b_qkv_lowp = self.b_qkv.to(dtype)
        # Compile (or find) the kernels for this head size now, not in the first step.
        kernels.attention_lib(self.head_dim)

    def _fuse_padded(self, params, dtype, device) -> None:
        """One projection matrix q | k | v | gate from separate tensors whose heads have
        ``key_dim`` (q, k) and ``value_dim`` (v) rows: every head is padded with rows of zeros to
        ``head_dim``, the output projection with columns of zeros, and the whole to a multiple of
        eight rows."""
        E, H, G, D = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim
        kd = int(params.get("key_dim", D))
        vd = int(params.get("value_dim", D))
        if not (0 < kd <= D and 0 < vd <= D):
            raise ValueError(f"key_dim={kd} and value_dim={vd} must lie within head_dim={D}")
        self.key_dim, self.value_dim = kd, vd

        def padded_heads(t, heads, size):
            t = t.reshape(heads, size, *t.shape[1:])
            if size == D:
                return t.reshape(heads * D, *t.shape[2:])
            out = t.new_zeros((heads, D) + tuple(t.shape[2:]))
            out[:, :size] = t
            return out.reshape(heads * D, *t.shape[2:])

        from_keys = bool(params.get("values_from_keys", False))
        if from_keys and vd != kd:
            raise ValueError(f"values_from_keys: value_dim={vd} must equal key_dim={kd}")
        # Values that are the unrotated keys: the projection has q and k rows only, and the kernel
        # that rotates k into its page copies the row's k, as it stands, into the value page.
        self.values_from_keys = from_keys
        if from_keys:
            if self.head_gate or not hasattr(self.position, "rotate_and_store") or getattr(
                    self.position, "layout", None) != "half":
                raise ValueError("values_from_keys goes with the rotary_half position part and no gate per head")
            self.qkv_width = self.q_size + self.kv_size
        pieces = [padded_heads(self.expect("q.weight", (H * kd, E)), H, kd),
                  padded_heads(self.expect("k.weight", (G * kd, E)), G, kd)]
        if not from_keys:
            pieces.append(padded_heads(self.expect("v.weight", (G * vd, E)), G, vd))
        bias = None
        if params.get("qkv_bias", False):
            bias = [padded_heads(self.expect("q.bias", (H * kd,)), H, kd),
                    padded_heads(self.expect("k.bias", (G * kd,)), G, kd)]
            if not from_keys:
                bias.append(padded_heads(self.expect("v.bias", (G * vd,)), G, vd))
        if self.head_gate:
            pieces.append(self.expect("gate.weight", (H, E)))
            if bias is not None:
                bias.append(bias[0].new_zeros(H))
        rows = sum(p.shape[0] for p in pieces)
        self.proj_width = -(-rows // 8) * 8
        if self.proj_width != rows:
            pieces.append(pieces[0].new_zeros(self.proj_width - rows, E))
            if bias is not None:
                bias.append(bias[0].new_zeros(self.proj_width - rows))
        self.w_qkv = torch.cat(pieces).contiguous()
        if bias is not None:
            self.b_qkv = torch.cat(bias).contiguous()
        w_out = self.expect("out.weight", (E, H * vd))
        if vd != D:
            wide = w_out.new_zeros(E, H, D)
            wide[:, :, :vd] = w_out.reshape(E, H, vd)
            w_out = wide.reshape(E, H * D).contiguous()
        self.w_out = w_out
        for name in ("q.weight", "k.weight", "v.weight", "q.bias", "k.bias", "v.bias", "gate.weight"):
            self.weights.pop(name, None)

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(paged=PagedCacheSpec(self.num_kv_heads, self.head_dim, self.window,
                                               keep_first=self.keep_first))

    def attention_signature(self):
        base = (self.num_kv_heads, self.num_heads // self.num_kv_heads, self.window, self.head_dim)
        return base + (self.keep_first, True) if self.anchored else base

    # The input is used by the QKV projection only, which can make the norm itself.
    accepts_pending_norm = True
    # Rows of tokens that belong to no sequence (padding of a rounded step) pass through like any
    # other row and are looked at by nobody.
    takes_padded_steps = True

    def forward(self, x, ctx, cache):
        T = ctx.num_tokens
        ws = ctx.workspace
        qkv = ws.get(f"attention.qkv{self.proj_width}", (ws.max_tokens, self.proj_width), self.dtype)
        group = ctx.groups[cache.group]
        k_cache, v_cache = (None, None) if cache.read_only else (cache.k, cache.v)
        # Projection, rotation and cache write in one kernel, where the position encoding
        # offers its tables and the kernel takes the shape (it says no otherwise).
        tables = None
        if _FUSE_ROPE and not self.values_from_keys:
            tables = getattr(self.position, "full_rotation_tables", lambda: None)()
        if tables is None or not qkv_rope_linear(
                x, self.w_qkv, self.b_qkv, qkv, T, ctx.status, ctx.positions, tables[0], tables[1],
                group.slot_mapping, k_cache, v_cache, self.num_heads, self.num_kv_heads):
            linear(x, self.w_qkv, self.b_qkv, qkv, T, self.b_qkv_lowp, status=ctx.status)
            if self.values_from_keys:
                self.position.rotate_and_store(qkv, ctx, group.slot_mapping, k_cache, v_cache,
                                               self.num_heads, self.num_kv_heads, values_from_keys=True)
            else:
                self.position.rotate_and_store(qkv, ctx, group.slot_mapping, k_cache, v_cache,
                                               self.num_heads, self.num_kv_heads)

        attn = ws.get(f"attention.out{self.q_size}", (ws.max_tokens, self.q_size), self.dtype)
        plan = ctx.attention_plan(cache.group, self.attention_signature())
        for kind, items, count in plan.launches:
            kernels.attention(
                kind, qkv, attn, cache.k, cache.v, group.block_tables, ctx.q_start, ctx.q_len,
                ctx.kv_len, items, count, plan.partial_o, plan.partial_lse, self.num_heads,
                self.num_kv_heads, self.head_dim, self.window, self.softmax_scale,
                merge_items=plan.merge_items, split_counters=plan.split_counters,
                status=ctx.status,
                cluster=(plan.cluster if kind == kernels.ATTN_BF16_NARROW else
                         getattr(plan, "tc_ctas_per_sm", 1) if kind == kernels.ATTN_BF16_TC else 1),
                layout_checked=getattr(plan, "checked", False),
                keep_first=self.keep_first, distance_bias=self.distance_bias, sink_zero=self.sink_zero,
                row_scale=self.row_scale,
            )
        if hasattr(plan, "checked"):
            plan.checked = True
        if plan.num_merges and plan.split_counters is None:
            kernels.attention_merge(
                attn, ctx.q_start, plan.merge_items, plan.num_merges, plan.partial_o,
                plan.partial_lse, self.num_heads, self.num_kv_heads, self.head_dim,
                max_rows=plan.merge_rows, sinks=self.sink,
            )
        if self.head_gate:
            kernels.head_gate(attn, qkv[:, self.qkv_width : self.qkv_width + self.num_heads], T,
                              self.num_heads, self.head_dim)

        if ctx.residual is not None and use_tensor_core_kernel(attn, self.w_out, T):
            # Few tokens: the projection is added straight into the float32 residual stream.
            mirror = getattr(ctx, "residual_mirror", None)
            linear(attn, self.w_out, None, ctx.residual, T, status=ctx.status, accumulate=True, mirror=mirror)
            if mirror is not None:
                ctx.residual_mirror_written = True
            return None
        out = ws.get("mixer.out", (ws.max_tokens, self.hidden_size), self.dtype)
        linear(attn, self.w_out, None, out, T, status=ctx.status)
        return out
