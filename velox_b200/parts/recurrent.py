"""Mixers that carry a state of fixed size from token to token, and the mixer that runs two
mixers side by side.

``gated_linear_recurrence``: two branches of ``width`` channels from one projection of the
input, ``y = act(W_y x + b_y)`` and ``u = conv(W_x x + b_x)`` (a causal convolution per channel);
u is cut into ``blocks`` equal parts and in part b ``r = sigmoid(A[b] u_b + a[b])``,
``i = sigmoid(I[b] u_b + c[b])``; with ``log a = -decay_scale * r * softplus(lam)`` the state is
``S <- a S + sqrt(1 - a^2) * i * u`` from ``S = 0`` (the first token is no special case) and the
result ``W_o (S * y)``.  (The recurrent block of De et al., "Griffin: Mixing Gated Linear
Recurrences with Local Attention for Efficient Language Models".)

``state_space``: one projection of the input gives ``z | x | B | C | dt``; x, B and C pass a
causal convolution per channel and SiLU; per head h (heads share B and C in ``groups``)
``dt = softplus(dt + dt_bias_h)``, ``S <- exp(-exp(A_log_h) dt) S + dt B x^T`` (S is state_size x
value_dim), ``y = S^T C + D_h x``; then ``y * silu(z)``, an RMS norm in ``norm_groups`` equal
parts times a weight, and W_o.  (The SSD layer of Dao and Gu, "Transformers are SSMs".)

Both keep, per request, the last ``taps - 1`` inputs of their convolution and the recurrent
state S in one float32 row of the slot-indexed state array, which starts at zero when a request
takes its slot.  Gates, decays, step sizes and S are float32 whatever the compute dtype; the
projections run in the compute dtype.

``delta_rule``: the generalized delta rule.  ``heads`` heads of ``dim`` channels; one projection
of the input gives ``r | k | v | g | a | w1`` (the last ``decay_rank`` rows are the first half of
the decay's two small matrices).  In float32, per head and key channel, the decay is
``w = exp(-decay_scale * sigmoid(W_w2 tanh(W_w1 x) + w0))`` and the removal rate ``a = sigmoid(W_a x
+ a_bias)``; with the unit key ``u = k / sqrt(sum(k^2) + key_eps)`` the state (``dim`` x ``dim`` per
head, float32) goes ``S <- diag(w) S - (a * u)(u^T S) + k v^T``, both middle terms reading the old
state, and the head's result is ``S^T r``, divided by its root mean square, times a weight over all
heads' channels, times ``sigmoid(g)``, then W_o.

``side_by_side``: two mixers read the same input; the result is ``scale * (rms_norm(left) * w_l
+ rms_norm(right) * w_r)`` over the model width, or, with ``join`` = "weighted_sum",
``left_scale * left + right_scale * right`` without norms.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import linear
from .base import CacheNeeds, Mixer, StateSpec
from .registry import part_class, register_part

_ACTS = {"none": kernels.ACT_NONE, "silu": kernels.ACT_SILU, "gelu_tanh": kernels.ACT_GELU_TANH,
         "relu_squared": kernels.ACT_RELU_SQUARED, "tanh": kernels.ACT_TANH}


def activation_code(name: str) -> int:
    try:
        return _ACTS[name]
    except KeyError:
        raise ValueError(f"unknown activation {name!r}; known: {sorted(_ACTS)}") from None


def _pad_rows(weight: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    rows = weight.shape[0]
    width = -(-rows // multiple) * multiple
    if width == rows:
        return weight
    return torch.cat([weight, weight.new_zeros((width - rows,) + tuple(weight.shape[1:]))]).contiguous()


def _lowered_rows(sums: torch.Tensor, ws, dtype, num_rows: int) -> torch.Tensor:
    """float32 rows in the compute dtype (for a block that has offered no stream to add into)."""
    if dtype == torch.float32:
        return sums
    out = ws.get("side_by_side.out", (ws.max_tokens, sums.shape[1]), dtype)
    kernels.cast_f32_to_bf16(sums, out, num_rows * sums.shape[1])
    return out


@register_part("mixer", "gated_linear_recurrence")
class GatedLinearRecurrence(Mixer):
    takes_padded_steps = True

    def __init__(self, params, weights, dtype, device, position=None) -> None:
        super().__init__(params, weights, dtype, device)
        self.hidden_size = E = int(params["hidden_size"])
        self.width = W = int(params["width"])
        self.blocks = int(params["blocks"])
        self.taps = int(params["conv_taps"])
        self.decay_scale = float(params.get("decay_scale", 8.0))
        self.branch_act = activation_code(params.get("branch_activation", "gelu_tanh"))
        if W % self.blocks != 0:
            raise ValueError(f"width={W} is not a multiple of blocks={self.blocks}")
        if self.taps < 1:
            raise ValueError("conv_taps must be at least 1")
        part = W // self.blocks
        # y | x in one projection.
        self.w_in = self.expect("in.weight", (2 * W, E))
        self.b_in = self.expect("in.bias", (2 * W,))
        self.in_width = -(-2 * W // 8) * 8
        self.w_in, self.b_in = _pad_rows(self.w_in), _pad_rows(self.b_in)
        self.b_in_lowp = self.b_in.to(dtype) if dtype != torch.float32 else None
        self.conv_w = self.expect("conv.weight", (W, self.taps))
        self.conv_b = self.expect("conv.bias", (W,))
        # The gate matrices are stored [block, out, in]; the kernel reads them [block, in, out].
        self.gate_a = self.expect("gate_a.weight", (self.blocks, part, part))
        self.gate_i = self.expect("gate_i.weight", (self.blocks, part, part))
        self.gate_a_t = self.gate_a.transpose(1, 2).contiguous()
        self.gate_i_t = self.gate_i.transpose(1, 2).contiguous()
        self.gate_a_b = self.expect("gate_a.bias", (self.blocks, part)).reshape(-1).contiguous()
        self.gate_i_b = self.expect("gate_i.bias", (self.blocks, part)).reshape(-1).contiguous()
        self.lam = self.expect("lam", (W,))
        self.w_out = self.expect("out.weight", (E, W))
        self.conv_elems = (self.taps - 1) * W
        kernels.mixers()

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(state=StateSpec(shape=(self.conv_elems + self.width,), dtype=torch.float32))

    def forward(self, x, ctx, cache):
        T, W = ctx.num_tokens, self.width
        ws = ctx.workspace
        if hasattr(x, "materialize"):
            x = x.materialize()
        proj = ws.get(f"recurrence.in{self.in_width}", (ws.max_tokens, self.in_width), self.dtype)
        linear(x, self.w_in, self.b_in, proj, T, self.b_in_lowp, status=ctx.status)
        u = ws.get(f"recurrence.u{W}", (ws.max_tokens, W), torch.float32)
        state = cache.state
        kernels.conv_tokens(proj[:, W : 2 * W], self.conv_w, self.conv_b, state[:, : max(self.conv_elems, 1)], u,
                            ctx.q_start, ctx.q_len, ctx.seq_slots, ctx.num_seqs, T, kernels.ACT_NONE)
        a = ws.get(f"recurrence.a{W}", (ws.max_tokens, W), torch.float32)
        b = ws.get(f"recurrence.b{W}", (ws.max_tokens, W), torch.float32)
        kernels.rglru_gates(u, self.gate_a_t, self.gate_a_b, self.gate_i_t, self.gate_i_b, self.lam,
                            self.decay_scale, a, b, T, w_a=self.gate_a, w_i=self.gate_i)
        gated = ws.get(f"recurrence.gated{W}", (ws.max_tokens, W), self.dtype)
        scratch = None
        if T > ctx.num_seqs:
            # Portions: long ones run in chunks of tokens side by side.
            size = kernels.rglru_scan_scratch(ws.max_tokens, state.shape[0], W)
            scratch = ws.get(f"recurrence.chunks{W}", (size,), torch.float32)
        kernels.rglru_scan(a, b, proj[:, :W], state[:, self.conv_elems : self.conv_elems + W], gated, ctx.q_start,
                           ctx.q_len, ctx.seq_slots, ctx.num_seqs, self.branch_act, scratch=scratch, num_tokens=T)
        out = ws.get(f"recurrence.out{self.hidden_size}", (ws.max_tokens, self.hidden_size), self.dtype)
        linear(gated, self.w_out, None, out, T, status=ctx.status)
        return out


@register_part("mixer", "state_space")
class StateSpace(Mixer):
    takes_padded_steps = True

    def __init__(self, params, weights, dtype, device, position=None) -> None:
        super().__init__(params, weights, dtype, device)
        self.hidden_size = E = int(params["hidden_size"])
        self.heads = H = int(params["heads"])
        self.value_dim = P = int(params["value_dim"])
        self.state_size = N = int(params["state_size"])
        self.groups = G = int(params["groups"])
        self.norm_groups = int(params.get("norm_groups", 1))
        self.taps = int(params["conv_taps"])
        self.eps = float(params["eps"])
        self.inner = inner = H * P
        if H % G != 0:
            raise ValueError(f"heads={H} is not a multiple of groups={G}")
        if inner % self.norm_groups != 0:
            raise ValueError(f"heads * value_dim = {inner} is not a multiple of norm_groups={self.norm_groups}")
        self.conv_channels = C = inner + 2 * G * N
        rows = 2 * inner + 2 * G * N + H
        self.w_in = _pad_rows(self.expect("in.weight", (rows, E)))
        self.in_width = self.w_in.shape[0]
        self.conv_w = self.expect("conv.weight", (C, self.taps))
        self.conv_b = self.expect("conv.bias", (C,))
        self.dt_bias = self.expect("dt_bias", (H,))
        self.a_log = self.expect("a_log", (H,))
        self.d_skip = self.expect("d", (H,))
        self.norm_w = self.expect("norm.weight", (inner,))
        self.w_out = self.expect("out.weight", (E, inner))
        self.conv_elems = (self.taps - 1) * C
        self.state_elems = H * N * P
        if N > 512:
            raise ValueError(f"state_size={N} is more than the scan kernel holds in a warp's registers (512)")
        kernels.mixers()

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(state=StateSpec(shape=(self.conv_elems + self.state_elems,), dtype=torch.float32))

    def forward(self, x, ctx, cache):
        T, inner, C = ctx.num_tokens, self.inner, self.conv_channels
        ws = ctx.workspace
        if hasattr(x, "materialize"):
            x = x.materialize()
        proj = ws.get(f"state_space.in{self.in_width}", (ws.max_tokens, self.in_width), self.dtype)
        linear(x, self.w_in, None, proj, T, status=ctx.status)
        xbc = ws.get(f"state_space.xbc{C}", (ws.max_tokens, C), torch.float32)
        state = cache.state
        kernels.conv_tokens(proj[:, inner : inner + C], self.conv_w, self.conv_b, state[:, : max(self.conv_elems, 1)],
                            xbc, ctx.q_start, ctx.q_len, ctx.seq_slots, ctx.num_seqs, T, kernels.ACT_SILU)
        y = ws.get(f"state_space.y{inner}", (ws.max_tokens, inner), torch.float32)
        scratch = None
        if T > ctx.num_seqs:
            # Portions: long ones run in chunks of tokens side by side.
            size = kernels.ssd_scan_scratch(ws.max_tokens, state.shape[0], self.heads, self.state_size, self.value_dim)
            scratch = ws.get(f"state_space.chunks{self.heads}_{self.state_size}_{self.value_dim}", (size,), torch.float32)
        kernels.ssd_scan(xbc, proj[:, inner + C : inner + C + self.heads], self.dt_bias, self.a_log, self.d_skip,
                         state[:, self.conv_elems : self.conv_elems + self.state_elems], y, self.heads, self.groups,
                         self.state_size, self.value_dim, ctx.q_start, ctx.q_len, ctx.seq_slots, ctx.num_seqs,
                         scratch=scratch, num_tokens=T)
        normed = ws.get(f"state_space.normed{inner}", (ws.max_tokens, inner), self.dtype)
        kernels.gated_group_norm(y, proj[:, :inner], self.norm_w, self.eps, self.norm_groups, normed, T)
        if ctx.residual is not None and self.dtype != torch.float32:
            from ..ops.linear import use_tensor_core_kernel

            if use_tensor_core_kernel(normed, self.w_out, T):
                linear(normed, self.w_out, None, ctx.residual, T, status=ctx.status, accumulate=True)
                return None
        out = ws.get(f"state_space.out{self.hidden_size}", (ws.max_tokens, self.hidden_size), self.dtype)
        linear(normed, self.w_out, None, out, T, status=ctx.status)
        return out


@register_part("mixer", "delta_rule")
class DeltaRule(Mixer):
    takes_padded_steps = True

    def __init__(self, params, weights, dtype, device, position=None) -> None:
        super().__init__(params, weights, dtype, device)
        self.hidden_size = E = int(params["hidden_size"])
        self.heads = H = int(params["heads"])
        self.dim = D = int(params["dim"])
        self.eps = float(params["eps"])
        self.decay_scale = float(params["decay_scale"])
        self.key_eps = float(params.get("key_eps", 1e-6))
        self.decay_rank = R = int(params["decay_rank"])
        if D > 512:
            raise ValueError(f"dim={D} is more than the scan kernel holds in a column's lanes (512)")
        self.inner = inner = H * D
        # r | k | v | g | a | w1 in one projection.  W_w1 is followed by rows of zeros up to a
        # multiple of eight, so tanh(W_w1 x) comes out padded with zeros to whole 16-byte rows; the
        # matching columns of W_w2 are zero.
        self.rank_padded = -(-R // 8) * 8
        w_in = self.expect("in.weight", (5 * inner + R, E))
        if self.rank_padded != R:
            w_in = torch.cat([w_in, w_in.new_zeros(self.rank_padded - R, E)])
        self.w_in = _pad_rows(w_in)
        self.in_width = self.w_in.shape[0]
        w2 = self.expect("decay_up.weight", (inner, R))
        if self.rank_padded != R:
            w2 = torch.cat([w2, w2.new_zeros(inner, self.rank_padded - R)], dim=1)
        self.w_decay_up = w2.contiguous()
        self.decay_bias = self.expect("decay_bias", (inner,))
        self.removal_bias = self.expect("removal_bias", (inner,))
        self.norm_w = self.expect("norm.weight", (inner,))
        self.w_out = self.expect("out.weight", (E, inner))
        self.state_elems = H * D * D
        kernels.mixers()

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(state=StateSpec(shape=(self.state_elems,), dtype=torch.float32))

    def forward(self, x, ctx, cache):
        T, inner = ctx.num_tokens, self.inner
        ws = ctx.workspace
        if hasattr(x, "materialize"):
            x = x.materialize()
        proj = ws.get(f"delta_rule.in{self.in_width}", (ws.max_tokens, self.in_width), self.dtype)
        linear(x, self.w_in, None, proj, T, status=ctx.status)
        # The decay's logits: the second small matrix on the tanh of the first one's product.
        bent = ws.get(f"delta_rule.bent{self.rank_padded}", (ws.max_tokens, self.rank_padded), self.dtype)
        kernels.act_rows(proj[:, 5 * inner : 5 * inner + self.rank_padded], bent, T, kernels.ACT_TANH)
        logits = ws.get(f"delta_rule.decay{inner}", (ws.max_tokens, inner), self.dtype)
        linear(bent, self.w_decay_up, None, logits, T, status=ctx.status)
        y = ws.get(f"delta_rule.y{inner}", (ws.max_tokens, inner), torch.float32)
        width = kernels.delta_rule_packed_width(self.heads, self.dim, self.dim)
        packed = ws.get(f"delta_rule.packed{width}", (ws.max_tokens, width), torch.float32)
        scratch = None
        if T >= 512:
            # Long steps: chunks of tokens side by side.
            size = kernels.delta_rule_chunk_scratch(ws.max_tokens, cache.state.shape[0], self.heads, self.dim, self.dim)
            scratch = ws.get(f"delta_rule.chunks{self.heads}_{self.dim}", (size,), torch.float32)
        kernels.delta_rule_scan(
            proj[:, :inner], proj[:, inner : 2 * inner], proj[:, 2 * inner : 3 * inner],
            proj[:, 4 * inner : 5 * inner], logits, self.decay_bias, self.removal_bias, self.decay_scale,
            self.key_eps, cache.state, y, self.heads, self.dim, self.dim, ctx.q_start, ctx.q_len, ctx.seq_slots,
            ctx.num_seqs, T, packed, ctx.status, chunk_scratch=scratch)
        normed = ws.get(f"delta_rule.normed{inner}", (ws.max_tokens, inner), self.dtype)
        kernels.gated_group_norm(y, proj[:, 3 * inner : 4 * inner], self.norm_w, self.eps, self.heads, normed, T,
                                 gate_after=True)
        out = ws.get(f"delta_rule.out{self.hidden_size}", (ws.max_tokens, self.hidden_size), self.dtype)
        linear(normed, self.w_out, None, out, T, status=ctx.status)
        return out


@register_part("mixer", "side_by_side")
class SideBySide(Mixer):
    """Two mixers on the same input.  ``params``: ``left`` and ``right``, each {kind, params};
    the weights of each child carry its prefix (``left.``, ``right.``); ``left.out_norm`` and
    ``right.out_norm`` are the weights of the RMS norms on the children's results; ``scale``
    (0.5: half the sum), ``eps``.  With ``join`` = "weighted_sum" there are no norms and the
    result is ``left_scale * left + right_scale * right``, summed in float32.  The children's
    caches are this part's: pages from the one, a state row from the other."""

    takes_padded_steps = True

    def __init__(self, params, weights, dtype, device, position=None) -> None:
        super().__init__(params, weights, dtype, device)
        self.hidden_size = int(params["hidden_size"])
        self.join = params.get("join", "normed_mean")
        if self.join not in ("normed_mean", "weighted_sum"):
            raise ValueError(f"side_by_side: join is 'normed_mean' or 'weighted_sum', not {self.join!r}")
        self.weighted = self.join == "weighted_sum"
        self.eps = float(params.get("eps", 0.0))
        self.scale = float(params.get("scale", 0.5))
        self.left_scale = float(params.get("left_scale", 1.0))
        self.right_scale = float(params.get("right_scale", 1.0))
        self.children = []
        for side in ("left", "right"):
            child = params[side]
            own = {name[len(side) + 1:]: t for name, t in weights.items()
                   if name.startswith(side + ".") and name != f"{side}.out_norm"}
            cls = part_class("mixer", child["kind"])
            self.children.append(cls(child["params"], own, dtype, device, position=position))
        if self.weighted:
            self.norm_left = self.norm_right = None
            kernels.heads()
        else:
            self.norm_left = self.expect("left.out_norm", (self.hidden_size,))
            self.norm_right = self.expect("right.out_norm", (self.hidden_size,))
        needs = [c.cache_needs() for c in self.children]
        if sum(n.paged is not None for n in needs) > 1 or sum(n.state is not None for n in needs) > 1:
            raise ValueError("side_by_side: at most one child may keep pages and at most one a state")
        self._needs = CacheNeeds(paged=next((n.paged for n in needs if n.paged is not None), None),
                                 state=next((n.state for n in needs if n.state is not None), None))
        self.takes_padded_steps = all(getattr(c, "takes_padded_steps", False) for c in self.children)
        kernels.mixers()

    def cache_needs(self) -> CacheNeeds:
        return self._needs

    def attention_signature(self):
        for child in self.children:
            signature = child.attention_signature()
            if signature is not None:
                return signature
        return None

    def forward(self, x, ctx, cache):
        T = ctx.num_tokens
        if hasattr(x, "materialize"):
            x = x.materialize()
        # The children's results are normed before they join the stream: they must not add
        # into it themselves.
        stream, ctx.residual = ctx.residual, None
        left = self.children[0].forward(x, ctx, cache)
        right = self.children[1].forward(x, ctx, cache)
        ctx.residual = stream
        if self.weighted:
            if stream is not None:
                kernels.add_rows(stream, left, right, T, self.left_scale, self.right_scale)
                return None
            sums = ctx.workspace.get("side_by_side.sums", (ctx.workspace.max_tokens, self.hidden_size), torch.float32)
            sums[:T].zero_()
            kernels.add_rows(sums, left, right, T, self.left_scale, self.right_scale)
            return _lowered_rows(sums, ctx.workspace, self.dtype, T)
        if stream is not None:
            kernels.dual_norm_mean(left, right, self.norm_left, self.norm_right, self.eps, self.scale, T,
                                   resid=stream)
            return None
        out = ctx.workspace.get("side_by_side.out", (ctx.workspace.max_tokens, self.hidden_size), self.dtype)
        kernels.dual_norm_mean(left, right, self.norm_left, self.norm_right, self.eps, self.scale, T, out=out)
        return out
