"""Arrangements of a layer's parts around the residual stream.

``pre_norm`` is the reference's decoder layer (src/decoder_layer.py:34-54):
``h = h + mixer(norm(h)); h = h + feed_forward(norm(h))``.  The adds are fused into the norm
that follows them, so a block leaves its last product pending in ``hidden.delta``.

``input_conv`` (block weight ``conv`` [width, taps]): the mixer does not read ``h_t = norm(x_t)``
but ``h_t + sum_j conv[:, j] * h_(t - taps + 1 + j)``, a causal convolution per channel over the
request's own tokens (zeros before its first).  The last ``taps - 1`` values of h of a request are
a float32 state row of the block.  Norm and convolution are one kernel.  A layer may then have
no feed-forward.
"""
from __future__ import annotations

import os

import torch

from ..ops import kernels
from .base import HiddenState, PendingSums
from .registry import register_part

# VELOX_B200_NO_NORM_FUSION=1 runs every norm as a kernel of its own (for bisecting).
_FUSE_NORMS = os.environ.get("VELOX_B200_NO_NORM_FUSION") != "1"


@register_part("block", "pre_norm")
class PreNormBlock:
    def __init__(self, mixer, feed_forward, norms, params=None, weights=None, dtype=None, device=None) -> None:
        params = dict(params or {})
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norm_mixer = norms["mixer"]
        self.norm_feed_forward = norms.get("feed_forward")
        if feed_forward is not None and self.norm_feed_forward is None:
            raise ValueError("a pre_norm block with a feed-forward needs its norm")
        self.conv = None
        if params.get("input_conv", False):
            if weights is None or "conv" not in weights:
                raise ValueError("a block with input_conv needs the weight 'conv'")
            self.conv = weights["conv"]
            if self.conv.dim() != 2 or self.conv.shape[0] != self.norm_mixer.size or not 1 <= self.conv.shape[1] <= 8:
                raise ValueError(f"the weight 'conv' has shape {tuple(self.conv.shape)}, expected "
                                 f"({self.norm_mixer.size}, taps) with 1 to 8 taps")
            if self.norm_mixer.center:
                raise ValueError("input_conv goes with an RMS norm")
            # The kernel reads the taps transposed: a tap of neighbouring channels is one load.
            self.conv_t = self.conv.to(torch.float32).t().contiguous()
            kernels.heads()

    def state_needs(self):
        """(taps - 1) rows of the model's width per request: the last inputs of the convolution."""
        if self.conv is None or self.conv.shape[1] < 2:
            return None
        from .base import StateSpec

        return StateSpec(((self.conv.shape[1] - 1) * self.norm_mixer.size,))

    def forward(self, hidden: HiddenState, ctx, cache) -> None:
        T = ctx.num_tokens
        ws = ctx.workspace
        normed = ws.get("block.normed", (ws.max_tokens, hidden.resid.shape[1]), self.mixer.dtype)
        # A part may add its product into the residual stream itself and return None.
        ctx.residual = hidden.resid
        # A feed-forward that adds into the stream while it still reads its input asks for a
        # copy of the rows; a mixer that adds its product itself can write it on the way.
        ctx.residual_mirror = None
        ctx.residual_mirror_written = False
        wants = getattr(self.feed_forward, "wants_residual_mirror", None)
        if wants is not None and wants(T, ctx):
            ctx.residual_mirror = ws.get("block.residual_mirror", (ws.max_tokens, hidden.resid.shape[1]), torch.float32)
        if self.conv is not None:
            if hidden.delta is not None:
                kernels.add_rows(hidden.resid, hidden.delta, None, T)
            kernels.norm_conv(hidden.resid, self.norm_mixer.weight, self.norm_mixer.eps, self.conv_t,
                              getattr(cache, "block_state", None), normed, T, ctx.q_start, ctx.q_len, ctx.seq_slots,
                              ctx.num_seqs)
            mixed = self.mixer.forward(normed, ctx, cache)
        else:
            mixed = self.mixer.forward(
                self._normed(self.norm_mixer, self.mixer, hidden.resid, hidden.delta, normed, T), ctx, cache)
        if self.feed_forward is None:
            hidden.delta = mixed
            ctx.residual = None
            ctx.residual_mirror = None
            return
        source = hidden.resid
        if mixed is None and ctx.residual_mirror is not None and ctx.residual_mirror_written:
            source = ctx.residual_mirror
        hidden.delta = self.feed_forward.forward(
            self._normed(self.norm_feed_forward, self.feed_forward, source, mixed, normed, T), ctx)
        ctx.residual = None
        ctx.residual_mirror = None

    @staticmethod
    def _normed(norm, consumer, resid, delta, out, num_rows):
        """The consumer's input: the norm's output, or, when nothing is waiting to be added and
        the consumer can take it, the norm itself for its first projection to make."""
        if _FUSE_NORMS and delta is None and getattr(consumer, "accepts_pending_norm", False):
            pending = norm.pending(resid, out, num_rows)
            if pending is not None:
                return pending
        norm.forward(resid, delta, out, num_rows)
        return out


@register_part("block", "post_norm")
class PostNormBlock:
    """The norm sits on each sublayer's result, not on its input:

        x <- x + norm_mixer(gate_1 * mixer(x));   x <- x + norm_ff(gate_2 * feed_forward(x))

    The sublayers read the stream itself (in the compute dtype).  ``gate_k = sigmoid(W x + b)``
    element by element when the part hands over side columns of its first projection
    (``ctx.side_output``: the block's W rides along as extra rows of that projection), else 1.
    A layer may have no feed-forward.

    ``depth_mix``: what goes on to the next layer is not the layer's result X_(e+1) but
    ``sum_{j <= e+1} w[j] X_j`` over the results of all layers so far (X_0 the embedding output),
    with the layer's own weights ``depth_mix.weight`` [e + 2].  The results are kept in one
    float32 store [entries + 2, tokens, width]: slot e + 1 is the layer's working copy of the
    stream (it starts as the layer's input and ends as X_(e+1)), the mixed rows go to slot e + 2,
    which is the next layer's working copy.  Each sublayer's gate, norm, add (and the mix after
    the last one) is one kernel, which also writes the outgoing rows in the compute dtype for
    the projection that reads them next.
    """

    def __init__(self, mixer, feed_forward, norms, params=None, weights=None, dtype=None, device=None) -> None:
        params = dict(params or {})
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norm_mixer = norms["mixer"]
        self.norm_feed_forward = norms.get("feed_forward")
        if feed_forward is not None and self.norm_feed_forward is None:
            raise ValueError("a post_norm block with a feed-forward needs its norm")
        self.depth_mix = bool(params.get("depth_mix", False))
        self.num_entries = int(params.get("num_entries", 0))
        self.mix_weight = None
        if self.depth_mix:
            if weights is None or "depth_mix.weight" not in weights:
                raise ValueError("a block with depth_mix needs the weight 'depth_mix.weight'")
            if self.num_entries < 1:
                raise ValueError("a block with depth_mix needs num_entries (the schedule's length)")
            self.mix_weight = weights["depth_mix.weight"]

    def _store(self, ws, width):
        return ws.get("block.results", (self.num_entries + 2, ws.max_tokens, width), torch.float32)

    def stream_home(self, ws):
        """Where the embedding output belongs: slot 0 of the store of results (None: anywhere)."""
        if not self.depth_mix:
            return None
        return self._store(ws, self.norm_mixer.size)[0]

    def forward(self, hidden: HiddenState, ctx, cache) -> None:
        T = ctx.num_tokens
        ws = ctx.workspace
        width = hidden.resid.shape[1]
        dtype = self.mixer.dtype
        if hidden.delta is not None:
            raise ValueError("a post_norm block takes a stream with nothing pending")
        x_in = hidden.resid
        work, store, mix_out, entry = x_in, None, None, ctx.entry_index
        if self.depth_mix:
            if self.mix_weight.numel() != entry + 2:
                raise ValueError(f"schedule entry {entry} mixes {entry + 2} results, its weight has {self.mix_weight.numel()}")
            store = self._store(ws, width)
            work, mix_out = store[entry + 1], store[entry + 2]
        lowp = None
        if dtype != torch.float32:
            lowp = ws.get("block.lowp", (ws.max_tokens, width), dtype)
            if hidden.lowp is None:
                kernels.cast_f32_to_bf16(x_in, lowp, T * width)
        source = x_in if lowp is None else lowp

        ctx.residual = None
        ctx.side_output = None
        mixed = self.mixer.forward(source, ctx, cache)
        last = self.feed_forward is None
        self._join(x_in, work, mixed, ctx.side_output, self.norm_mixer, T, lowp, store, mix_out, last)
        if not last:
            source = work if lowp is None else lowp
            ctx.side_output = None
            ctx.takes_pending_sums = lowp is not None
            product = self.feed_forward.forward(source, ctx)
            ctx.takes_pending_sums = False
            self._join(work, work, product, ctx.side_output, self.norm_feed_forward, T, lowp, store, mix_out, True)
        ctx.side_output = None
        hidden.resid = mix_out if self.depth_mix else work
        hidden.delta = None
        hidden.lowp = lowp

    def _join(self, resid_in, resid_out, delta, gate, norm, num_rows, lowp, store, mix_out, last) -> None:
        mixing = self.depth_mix and last
        sums = bias = None
        if isinstance(delta, PendingSums):
            sums, bias, delta = delta.sums, delta.bias, None
        kernels.gated_norm_add(
            resid_in, resid_out, delta, gate, norm.weight, norm.eps, norm.center, num_rows, lowp_out=lowp,
            history=store if mixing else None, mix_weights=self.mix_weight if mixing else None,
            mix_out=mix_out if mixing else None, sums=sums, sums_bias=bias,
            compute_dtype=None if sums is None else lowp.dtype,
        )


@register_part("block", "parallel")
class ParallelBlock:
    """Both sublayers read the same rows x:  ``x <- x + (mixer(norm_a(x)) + feed_forward(norm_b(x)))``.
    With one norm (``norms["input"]`` alone) both read its output; with ``norms["feed_forward"]``
    as well, each sublayer has its own norm of the same x.  A layer may have no feed-forward.
    The sums are float32: a part adds its product into the stream itself where it can
    (``ctx.residual``), what it returns instead is added here, and the last product may stay
    pending for the next norm to add.

    ``token_shift`` (block weight ``shift`` [width]): the mixer does not read ``h_t = norm_a(x_t)``
    but ``h_t + (h_(t-1) - h_t) * shift`` with the request's previous token's h (as the norm
    made it; zeros before the first token).  The last h of a request is a float32 state row of
    the block.  Norms and shift are one kernel, which reads x once.
    """

    def __init__(self, mixer, feed_forward, norms, params=None, weights=None, dtype=None, device=None) -> None:
        params = dict(params or {})
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norm = norms["input"]
        self.norm_feed_forward = norms.get("feed_forward")
        self.shift = None
        if params.get("token_shift", False):
            if weights is None or "shift" not in weights:
                raise ValueError("a block with token_shift needs the weight 'shift'")
            self.shift = weights["shift"]
            if tuple(self.shift.shape) != (self.norm.size,):
                raise ValueError(f"the weight 'shift' has shape {tuple(self.shift.shape)}, expected ({self.norm.size},)")
        self.two_outputs = self.norm_feed_forward is not None and feed_forward is not None
        if self.two_outputs and (self.norm_feed_forward.eps != self.norm.eps or self.norm_feed_forward.center
                                 or self.norm.center):
            raise ValueError("a parallel block's two norms are RMS norms with one eps")
        if self.shift is not None or self.two_outputs:
            kernels.heads()

    def state_needs(self):
        """A row of the model's width per request: the previous token's normed input."""
        if self.shift is None:
            return None
        from .base import StateSpec

        return StateSpec((self.norm.size,))

    def forward(self, hidden: HiddenState, ctx, cache) -> None:
        T = ctx.num_tokens
        ws = ctx.workspace
        width = hidden.resid.shape[1]
        normed = ws.get("block.normed", (ws.max_tokens, width), self.mixer.dtype)
        for_feed_forward = normed
        if self.shift is None and not self.two_outputs:
            self.norm.forward(hidden.resid, hidden.delta, normed, T)
        else:
            if hidden.delta is not None:
                kernels.add_rows(hidden.resid, hidden.delta, None, T)
            if self.two_outputs:
                for_feed_forward = ws.get("block.normed_b", (ws.max_tokens, width), self.mixer.dtype)
            kernels.norm_shift(
                hidden.resid, self.norm.weight, self.norm.eps, normed, T, ctx.q_start, ctx.q_len, ctx.seq_slots,
                ctx.num_seqs, weight2=self.norm_feed_forward.weight if self.two_outputs else None,
                out2=for_feed_forward if self.two_outputs else None, shift=self.shift,
                state=cache.block_state if self.shift is not None else None)
        hidden.delta = None
        ctx.residual = hidden.resid
        ctx.residual_mirror = None
        ctx.residual_mirror_written = False
        mixed = self.mixer.forward(normed, ctx, cache)
        if self.feed_forward is None:
            hidden.delta = mixed
        else:
            if self.shift is None and not self.two_outputs:
                if mixed is not None:
                    kernels.residual_add(hidden.resid, mixed, T)
                hidden.delta = self.feed_forward.forward(for_feed_forward, ctx)
            else:
                # Both products were made from the same rows, so they go into the stream together,
                # in one pass over it; nothing stays pending for the next block's norms.
                product = self.feed_forward.forward(for_feed_forward, ctx)
                if mixed is not None:
                    kernels.add_rows(hidden.resid, mixed, product, T)
                else:
                    hidden.delta = product
        ctx.residual = None
