"""Dense feed-forward parts.  ``swiglu`` is the reference's MLP: ``down(silu(gate(x)) * up(x))``
with gate and up fused into one matrix whose first half is gate, and no biases
(src/mlp.py:9-15).  SiLU and the product are computed in float32 and rounded once (the reference
rounds to the model dtype between the two)."""
from __future__ import annotations

import math
import os

import torch

from ..ops import kernels
from ..ops.linear import DETERMINISTIC, choose_splits, linear, swiglu_linear, use_tensor_core_kernel
from .base import FeedForward, PendingSums
from .registry import register_part


# VELOX_B200_NO_LIBRARY_GROUPED=1 keeps the experts of long steps on this package's own tiled
# kernel (for comparison, and for a torch without a grouped product).
_LIBRARY_GROUPED = os.environ.get("VELOX_B200_NO_LIBRARY_GROUPED") != "1"

# VELOX_B200_NO_MLP_FUSION=1 keeps the two projections of a small step as kernels of their own
# (for bisecting; the fused kernel's sum over the inner width has no fixed order).
_FUSE_MLP = os.environ.get("VELOX_B200_NO_MLP_FUSION") != "1" and not DETERMINISTIC


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, params, weights, dtype, device) -> None:
        super().__init__(params, weights, dtype, device)
        self.hidden_size = int(params["hidden_size"])
        self.intermediate_size = int(params["intermediate_size"])
        self.w_gate_up = self.expect("gate_up.weight", (2 * self.intermediate_size, self.hidden_size))
        self.w_down = self.expect("down.weight", (self.hidden_size, self.intermediate_size))

    # The input is used by the gate|up projection only, which can make the norm itself.
    accepts_pending_norm = True
    # Rows of tokens that belong to no sequence (padding of a rounded step) pass through like any
    # other row and are looked at by nobody.
    takes_padded_steps = True

    def _fusable(self, T, ctx) -> bool:
        return (_FUSE_MLP and 0 < T <= kernels.MLP_FUSED_MAX_TOKENS and self.dtype == torch.bfloat16
                and ctx.status is not None and self.hidden_size % 128 == 0 and self.intermediate_size % 64 == 0)

    def wants_residual_mirror(self, T, ctx) -> bool:
        """With few tokens the whole feed-forward is one kernel whose CTAs add their shares into
        the residual stream while others still read their input rows: it reads a copy."""
        return self._fusable(T, ctx)

    def forward(self, x, ctx):
        T = ctx.num_tokens
        ws = ctx.workspace
        if (self._fusable(T, ctx) and ctx.residual is not None and getattr(x, "resid", None) is not None
                and x.resid.data_ptr() != ctx.residual.data_ptr() and x.resid.dtype == torch.float32):
            if kernels.mlp_fused(x.resid, x.weight, x.eps, self.w_gate_up, self.w_down, ctx.residual, T, ctx.status):
                return None
        act = ws.get("swiglu.act", (ws.max_tokens, self.intermediate_size), self.dtype)
        if use_tensor_core_kernel(x, self.w_gate_up, T) and use_tensor_core_kernel(act, self.w_down, T):
            # Few tokens: SiLU(gate) * up in the projection's epilogue, then the down projection
            # added straight into the float32 residual stream.
            swiglu_linear(x, self.w_gate_up, act, T, ctx.status)
            if ctx.residual is not None:
                linear(act, self.w_down, None, ctx.residual, T, status=ctx.status, accumulate=True)
                return None
            out = ws.get("feed_forward.out", (ws.max_tokens, self.hidden_size), self.dtype)
            linear(act, self.w_down, None, out, T, status=ctx.status)
            return out
        gate_up = ws.get("swiglu.gate_up", (ws.max_tokens, 2 * self.intermediate_size), self.dtype)
        linear(x, self.w_gate_up, None, gate_up, T)
        kernels.swiglu(gate_up, act, T)
        out = ws.get("feed_forward.out", (ws.max_tokens, self.hidden_size), self.dtype)
        linear(act, self.w_down, None, out, T)
        return out


def _softplus(value: float) -> float:
    return max(value, 0.0) + math.log1p(math.exp(-abs(value)))


@register_part("feed_forward", "dense_xielu")
class DenseXielu(FeedForward):
    """``down(act(up(x)))`` with biases on both projections and the xIELU activation with two
    learned numbers p, q (``act`` weight): ``z > 0: softplus(p) z^2 + z / 2``, ``z <= 0:
    (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2``, computed in float32.

    ``side_rows`` > 0: the first rows of ``up.weight`` / ``up.bias`` are not the feed-forward's;
    their products belong to the block around it (a gate over the result) and are handed over
    as ``ctx.side_output``, so the block's projection of the same input rides along."""

    takes_padded_steps = True

    def __init__(self, params, weights, dtype, device) -> None:
        super().__init__(params, weights, dtype, device)
        self.hidden_size = int(params["hidden_size"])
        self.intermediate_size = int(params["intermediate_size"])
        self.side_rows = int(params.get("side_rows", 0))
        rows = self.intermediate_size + self.side_rows
        self.w_up = self.expect("up.weight", (rows, self.hidden_size))
        self.b_up = self.expect("up.bias", (rows,))
        # Rows of zeros up to a multiple of eight (16-byte output rows in bfloat16).
        self.up_width = -(-rows // 8) * 8
        if self.up_width != rows:
            self.w_up = torch.cat([self.w_up, self.w_up.new_zeros(self.up_width - rows, self.hidden_size)]).contiguous()
            self.b_up = torch.cat([self.b_up, self.b_up.new_zeros(self.up_width - rows)]).contiguous()
        self.w_down = self.expect("down.weight", (self.hidden_size, self.intermediate_size))
        self.b_down = self.expect("down.bias", (self.hidden_size,))
        self.b_up_lowp = self.b_up.to(dtype) if dtype != torch.float32 else None
        self.b_down_lowp = self.b_down.to(dtype) if dtype != torch.float32 else None
        p, q = (float(v) for v in self.expect("act", (2,)).tolist())
        self.a_pos = _softplus(p)
        self.a_neg = 0.5 + _softplus(q)

    def forward(self, x, ctx):
        T = ctx.num_tokens
        ws = ctx.workspace
        rows = self.up_width
        up = ws.get(f"dense.up{rows}", (ws.max_tokens, rows), self.dtype)
        ctx.side_output = up[:, : self.side_rows] if self.side_rows else None
        act = ws.get(f"dense.act{self.intermediate_size}", (ws.max_tokens, self.intermediate_size), self.dtype)
        # Few tokens: the activation is made in the projection's epilogue (the rows of zeros at
        # the end of a padded matrix are left out of that launch).
        fused = (ctx.status is not None and use_tensor_core_kernel(x, self.w_up, T)
                 and kernels.gemm_bf16_xielu(x, self.w_up[: self.side_rows + self.intermediate_size],
                                             self.b_up, up, act, self.side_rows, self.a_pos, self.a_neg, T,
                                             ctx.status, splits=choose_splits(self.up_width, self.hidden_size, T)))
        if not fused:
            linear(x, self.w_up, self.b_up, up, T, self.b_up_lowp, status=ctx.status)
            kernels.xielu(up[:, self.side_rows :], act, T, self.a_pos, self.a_neg)
        if (getattr(ctx, "takes_pending_sums", False) and ctx.status is not None
                and use_tensor_core_kernel(act, self.w_down, T)):
            # Few tokens and a block that can take it: the down projection's K is cut into chunks
            # of independent CTAs that add their shares into float32 rows (zero before, and set to
            # zero again by the block's join kernel, which also adds the bias).
            sums = ws.get("dense.sums", (ws.max_tokens, self.hidden_size), torch.float32)
            linear(act, self.w_down, None, sums, T, status=ctx.status, accumulate=True)
            return PendingSums(sums, self.b_down)
        out = ws.get("feed_forward.out", (ws.max_tokens, self.hidden_size), self.dtype)
        linear(act, self.w_down, self.b_down, out, T, self.b_down_lowp, status=ctx.status)
        return out


def _pad_to(t: torch.Tensor, dim: int, multiple: int = 8) -> torch.Tensor:
    size = t.shape[dim]
    wide = -(-size // multiple) * multiple
    if wide == size:
        return t.contiguous()
    shape = list(t.shape)
    shape[dim] = wide - size
    return torch.cat([t, t.new_zeros(shape)], dim=dim).contiguous()


@register_part("feed_forward", "dense_act")
class DenseAct(FeedForward):
    """``down(act(up(x)))`` without biases; ``activation`` is ``gelu_tanh`` (0.5 z (1 + tanh(
    sqrt(2/pi) (z + 0.044715 z^3)))), ``relu_squared`` or ``silu``, computed in float32.

    ``gate_rows`` > 0: that many further rows of ``up.weight`` (behind the feed-forward's own) are
    a gate over the result: the part's product is ``sigmoid(gate . x) * down(...)``, one number per
    token (``gate_rows`` is 1), added to the residual stream by the part itself."""

    takes_padded_steps = True

    def __init__(self, params, weights, dtype, device) -> None:
        super().__init__(params, weights, dtype, device)
        from .recurrent import activation_code

        self.hidden_size = E = int(params["hidden_size"])
        self.intermediate_size = F = int(params["intermediate_size"])
        self.act = activation_code(params.get("activation", "gelu_tanh"))
        self.gate_rows = int(params.get("gate_rows", 0))
        if self.gate_rows not in (0, 1):
            raise ValueError("dense_act: gate_rows is 0 or 1")
        self.w_up = _pad_to(self.expect("up.weight", (F + self.gate_rows, E)), 0)
        self.up_width = self.w_up.shape[0]
        # The activated rows are padded with zeros to whole 16-byte rows; the matching columns of
        # the down projection are zero.
        self.w_down = _pad_to(self.expect("down.weight", (E, F)), 1)
        self.act_width = self.w_down.shape[1]
        kernels.mixers()

    def forward(self, x, ctx):
        T = ctx.num_tokens
        ws = ctx.workspace
        if hasattr(x, "materialize"):
            x = x.materialize()
        up = ws.get(f"dense_act.up{self.up_width}", (ws.max_tokens, self.up_width), self.dtype)
        linear(x, self.w_up, None, up, T, status=ctx.status)
        act = ws.get(f"dense_act.act{self.intermediate_size}_{self.act_width}", (ws.max_tokens, self.act_width),
                     self.dtype)
        kernels.act_rows(up[:, : self.intermediate_size], act[:, : self.intermediate_size], T, self.act)
        if self.gate_rows:
            down = ws.get(f"dense_act.down{self.hidden_size}", (ws.max_tokens, self.hidden_size), self.dtype)
            linear(act, self.w_down, None, down, T, status=ctx.status)
            gate = up[:, self.intermediate_size : self.intermediate_size + 1]
            if ctx.residual is not None:
                kernels.gated_rows_add(ctx.residual, down, gate, T)
                return None
            sums = ws.get(f"dense_act.sums{self.hidden_size}", (ws.max_tokens, self.hidden_size), torch.float32)
            sums[:T].zero_()
            kernels.gated_rows_add(sums, down, gate, T)
            return _lowered(sums, ws, self.dtype, T, "dense_act.gated")
        if (ctx.residual is not None and ctx.status is not None and self.dtype != torch.float32
                and use_tensor_core_kernel(act, self.w_down, T)):
            linear(act, self.w_down, None, ctx.residual, T, status=ctx.status, accumulate=True)
            return None
        out = ws.get("feed_forward.out", (ws.max_tokens, self.hidden_size), self.dtype)
        linear(act, self.w_down, None, out, T, status=ctx.status)
        return out


@register_part("feed_forward", "clamped_glu")
class ClampedGLU(FeedForward):
    """A gated feed-forward with clamps and biases:

        g = min(W_g x + b_g, limit);   u = clamp(W_u x + b_u, -limit, limit)
        y = g * sigmoid(alpha * (g + cubic * g^3)) * (u + up_shift);   out = W_d y + b_d

    ``gate_up.weight`` holds the gate rows first, then the up rows (and ``gate_up.bias`` alike);
    ``limit`` 0 means no clamps; ``alpha``, ``cubic`` and ``up_shift`` default to 1, 0 and 0, which is
    SwiGLU; ``alpha`` = 2 sqrt(2 / pi) with ``cubic`` = 0.044715 is the tanh form of GELU on the gate,
    ``g / 2 * (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3)))``, because ``(1 + tanh y) / 2 = sigmoid(2 y)``.
    ``biases`` false: the part has no bias vectors.
    The activation is float32.  The inner width need not be a multiple of anything: both halves
    are padded with rows of zeros to a multiple of eight, which produce y = 0."""

    takes_padded_steps = True

    def __init__(self, params, weights, dtype, device) -> None:
        super().__init__(params, weights, dtype, device)
        self.hidden_size = E = int(params["hidden_size"])
        self.intermediate_size = F = int(params["intermediate_size"])
        self.limit = float(params.get("limit") or 0.0)
        self.alpha = float(params.get("alpha", 1.0))
        self.up_shift = float(params.get("up_shift", 0.0))
        self.cubic = float(params.get("cubic", 0.0))
        if self.limit < 0.0:
            raise ValueError(f"clamped_glu: limit={self.limit} must not be negative")
        w = self.expect("gate_up.weight", (2 * F, E))
        b = self.expect("gate_up.bias", (2 * F,)) if params.get("biases", True) else None
        self.inner = Fp = -(-F // 8) * 8
        self.w_gate_up = torch.cat([_pad_to(w[:F], 0), _pad_to(w[F:], 0)]).contiguous()
        self.b_gate_up = None if b is None else torch.cat([_pad_to(b[:F], 0), _pad_to(b[F:], 0)]).contiguous()
        self.w_down = _pad_to(self.expect("down.weight", (E, F)), 1)
        self.b_down = self.expect("down.bias", (E,)) if params.get("biases", True) else None
        lowp = dtype != torch.float32
        self.b_gate_up_lowp = self.b_gate_up.to(dtype) if lowp and self.b_gate_up is not None else None
        self.b_down_lowp = self.b_down.to(dtype) if lowp and self.b_down is not None else None
        self.weights.pop("gate_up.weight", None)
        kernels.heads()

    def forward(self, x, ctx):
        T = ctx.num_tokens
        ws = ctx.workspace
        if hasattr(x, "materialize"):
            x = x.materialize()
        Fp = self.inner
        act = ws.get(f"clamped_glu.act{Fp}", (ws.max_tokens, Fp), self.dtype)
        if ctx.status is not None and use_tensor_core_kernel(x, self.w_gate_up, T):
            # Few tokens: biases, clamps and activation in the projection's epilogue.
            kernels.gemm_bf16_glu(x, self.w_gate_up, self.b_gate_up, act, T, self.limit, self.alpha, self.up_shift,
                                  ctx.status, cubic=self.cubic)
        else:
            gate_up = ws.get(f"clamped_glu.gate_up{2 * Fp}", (ws.max_tokens, 2 * Fp), self.dtype)
            linear(x, self.w_gate_up, self.b_gate_up, gate_up, T, self.b_gate_up_lowp, status=ctx.status)
            kernels.clamped_glu(gate_up, act, T, Fp, self.limit, self.alpha, self.up_shift, cubic=self.cubic)
        if (ctx.residual is not None and ctx.status is not None and self.dtype != torch.float32
                and use_tensor_core_kernel(act, self.w_down, T)):
            # Few tokens: the down projection (and its bias) goes straight into the float32 stream.
            linear(act, self.w_down, self.b_down, ctx.residual, T, status=ctx.status, accumulate=True)
            return None
        out = ws.get("feed_forward.out", (ws.max_tokens, self.hidden_size), self.dtype)
        linear(act, self.w_down, self.b_down, out, T, self.b_down_lowp, status=ctx.status)
        return out


def _lowered(sums: torch.Tensor, ws, dtype, num_rows: int, name: str) -> torch.Tensor:
    """float32 rows in the compute dtype (for a block that has offered no stream to add into)."""
    if dtype == torch.float32:
        return sums
    out = ws.get(name, tuple(sums.shape), dtype)
    kernels.cast_f32_to_bf16(sums, out, num_rows * sums.shape[1])
    return out


@register_part("feed_forward", "table_experts")
class TableExperts(FeedForward):
    """``experts`` small feed-forwards ``down_e(relu(up_e(x))^2)`` without biases, of which every
    token uses ``top``: row ``token id`` of an integer ``table`` [vocab, top] names them (there
    is no router), each with weight 1 / top.  ``up.weight`` / ``down.weight`` are the experts'
    matrices one after the other.  ``shared``: parameters of a ``dense_act`` part that runs for
    every token beside them (its weights carry the prefix ``shared.``).

    The part adds its result into the float32 residual stream itself."""

    takes_padded_steps = True

    def __init__(self, params, weights, dtype, device) -> None:
        super().__init__(params, weights, dtype, device)
        self.hidden_size = E = int(params["hidden_size"])
        self.experts = X = int(params["experts"])
        self.top = int(params["top"])
        self.expert_ff = F = int(params["expert_ff"])
        self.vocab_size = int(params["vocab_size"])
        if not 0 < self.top <= X:
            raise ValueError(f"top={self.top} must lie within experts={X}")
        self.w_up = self.expect("up.weight", (X * F, E)).view(X, F, E)
        self.w_down = self.expect("down.weight", (X * E, F)).view(X, E, F)
        self.table = self.expect("table", (self.vocab_size, self.top))
        self.shared = None
        if params.get("shared"):
            own = {name[len("shared."):]: t for name, t in weights.items() if name.startswith("shared.")}
            self.shared = DenseAct(params["shared"], own, dtype, device)
        kernels.mixers()

    # Steps with more tokens than this run the experts as tiled tensor-core products over the
    # (token, expert) pairs ordered by expert; shorter ones as matrix-vector products spread over
    # the grid (every pair then reads its expert's matrices once).
    GROUPED_FROM_TOKENS = 48
    # ... and beyond the projections' small-step limit as the library's grouped product (one launch
    # over all experts, the runs' ends read on the device), where torch has one.
    LIBRARY_FROM_TOKENS = 256

    def _experts(self, x, ctx, target, T) -> None:
        ws = ctx.workspace
        ids, fed = ctx.token_ids, getattr(ctx, "fed_tokens", None)
        X, F, E = self.experts, self.expert_ff, self.hidden_size
        if self.dtype == torch.bfloat16 and T > self.LIBRARY_FROM_TOKENS and _LIBRARY_GROUPED:
            # Long steps: the projections' rule (library products beyond the small-step limit).
            places = kernels.grouped_places(T, self.top, X)
            most = kernels.grouped_places(ws.max_tokens, self.top, X)
            route = ws.get(f"table_experts.route{most}", (2 * most + ws.max_tokens * self.top,), torch.int32)
            ends = ws.get(f"table_experts.ends{X}", (X,), torch.int32)
            a_rows = ws.get(f"table_experts.gathered{E}", (most, E), torch.bfloat16)
            if kernels.table_experts_library(x, ids, fed, self.table, self.w_up, self.w_down, route, ends,
                                             a_rows[:places], target, T, ctx.status):
                return
        if self.dtype == torch.bfloat16 and T > self.GROUPED_FROM_TOKENS:
            places = kernels.grouped_places(ws.max_tokens, self.top, X)
            route = ws.get(f"table_experts.route{places}", (2 * places + ws.max_tokens * self.top,), torch.int32)
            act = ws.get(f"table_experts.act{F}", (places, F), torch.bfloat16)
            rows = ws.get(f"table_experts.rows{E}", (places, E), torch.float32)
            if kernels.table_experts_grouped(x, ids, fed, self.table, self.w_up, self.w_down, route, act, rows,
                                             target, T, ctx.status):
                return
        act = ws.get(f"table_experts.act32_{F}", (ws.max_tokens * self.top * F,), torch.float32)
        if kernels.table_experts_rows(x, ids, fed, self.table, self.w_up, self.w_down, act, target, T, ctx.status):
            return
        kernels.table_experts(x, ids, fed, self.table, self.w_up, self.w_down, target, T, ctx.status)

    def forward(self, x, ctx):
        T = ctx.num_tokens
        ws = ctx.workspace
        if hasattr(x, "materialize"):
            x = x.materialize()
        stream = ctx.residual
        target = stream
        if target is None:
            target = ws.get(f"table_experts.sums{self.hidden_size}", (ws.max_tokens, self.hidden_size), torch.float32)
            target[:T].zero_()
        self._experts(x, ctx, target, T)
        if self.shared is not None:
            ctx.residual = target
            product = self.shared.forward(x, ctx)
            ctx.residual = stream
            if product is not None:
                kernels.residual_add(target, product, T)
        if stream is not None:
            return None
        return _lowered(target, ws, self.dtype, T, "table_experts.out")
