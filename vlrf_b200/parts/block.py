"""Blocks: how a layer arranges its norm, mixer and feed-forward around the residual stream."""
from __future__ import annotations

import torch

from .context import StepContext
from .registry import register_part


@register_part("block", "pre_norm")
class PreNormBlock:
    """x += mixer(norm1(x)); x += ffn(norm2(x)) (reference: include/model/transformer_block.hpp:149-159).
    The residual stream x stays float32; the normed rows are in the activation dtype.

    A first norm that keeps something per sequence (one with a `cache_need` of its own, such as a norm with a token
    shift) is given the step and its state; what it keeps is the last entry of the block's need, behind the mixer's."""

    def __init__(self, norm1, mixer, norm2, feed_forward):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward
        self._norm_keeps = hasattr(norm1, "cache_need")

    def cache_need(self):
        need = self.mixer.cache_need()
        if not self._norm_keeps:
            return need
        own = self.norm1.cache_need()
        if need is None:
            return (own,)
        return (*need, own) if isinstance(need, tuple) else (need, own)

    def _views(self, view):
        """(the mixer's view, the first norm's state) of a block whose first norm keeps something."""
        from ..cache import CacheView
        parts = view.parts
        if len(parts) == 1:
            return None, parts[0].state
        if len(parts) == 2:
            return parts[0], parts[1].state
        return CacheView(tuple(p.need for p in parts[:-1]), parts=parts[:-1]), parts[-1].state

    @property
    def leaves_row_stats(self) -> bool:
        """Whether the step's row statistics are true after this block: its last part says (see forward)."""
        return bool(getattr(self.feed_forward, "leaves_row_stats", False))

    def emit_decode(self, program, x: torch.Tensor, view, writes_cache: bool = True) -> None:
        """This block's decode step as operations of a decode program: possible when the mixer and the
        feed-forward can state theirs (they get the norm to fuse, as in `forward`)."""
        from .program import NotFusable
        if self._norm_keeps:
            raise NotFusable("a norm that keeps a state is not an operation of the decode program")
        for part in (self.mixer, self.feed_forward):
            if not hasattr(part, "emit_decode"):
                raise NotFusable(f"{type(part).__name__} has no emit_decode")
        self.mixer.emit_decode(program, x, self.norm1, view, writes_cache)
        self.feed_forward.emit_decode(program, x, self.norm2)

    def forward(self, x: torch.Tensor, ctx: StepContext, view, writes_cache: bool = True) -> None:
        if self._norm_keeps:
            if not writes_cache:
                raise ValueError("PreNormBlock: a layer whose norm keeps a state cannot run on another layer's cache")
            mixer_view, kept = self._views(view)
            h = ctx.ws.get("block_normed", ctx.n_tokens, x.shape[1], ctx.act_dtype)
            self.mixer.forward(self.norm1(x, h, ctx=ctx, state=kept), x, ctx, mixer_view, writes_cache)
        elif getattr(self.mixer, "fuses_norm", False):
            self.mixer.forward(None, x, ctx, view, writes_cache, norm=self.norm1)
        else:
            h = ctx.ws.get("block_normed", ctx.n_tokens, x.shape[1], ctx.act_dtype)
            self.mixer.forward(self.norm1(x, h), x, ctx, view, writes_cache)
        # What is known about the residual rows (their statistics, for a fused LayerNorm) is true only if the part
        # that just rewrote them says so; a part with kernels of its own need not know that such a thing exists.
        if not getattr(self.mixer, "leaves_row_stats", False):
            ctx.ws.row_stats.forget()
        if self.feed_forward is None:          # a layer without a feed-forward
            return
        if getattr(self.feed_forward, "fuses_norm", False):
            self.feed_forward.forward(None, x, ctx, norm=self.norm2)
        else:
            h = ctx.ws.get("block_normed", ctx.n_tokens, x.shape[1], ctx.act_dtype)
            self.feed_forward.forward(self.norm2(x, h), x, ctx)
        if not getattr(self.feed_forward, "leaves_row_stats", False):
            ctx.ws.row_stats.forget()


@register_part("block", "sublayer_norm")
class SublayerNormBlock:
    """x += norm1(mixer(x)); x += norm2(ffn(x)): the norm acts on each sublayer's output, and the sublayers read the
    residual stream itself (rounded to the activation dtype where that is not float32).  The stream and the norm are
    float32; the sublayer writes its float32 output into scratch (`accumulate=False`), and the norm adds to x.
    Either sublayer may be absent (None)."""

    leaves_row_stats = False

    def __init__(self, norm1, mixer, norm2, feed_forward):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def cache_need(self):
        return self.mixer.cache_need() if self.mixer is not None else None

    #: the block leaves `ws.input_cast` true (see `_input`); the model forgets it after layers that do not say so
    leaves_input_cast = True

    def _input(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """What a sublayer reads: x itself in the 32-bit engine, else its rounding to the activation dtype.  The norm
        that last added to x has written that rounding already (`ws.input_cast` names the rows it is of); only the
        first sublayer after something else wrote x (the embedding) casts."""
        if ctx.act_dtype == torch.float32:
            return x
        from ..csrc import ops
        h = ctx.ws.get("block_input", ctx.n_tokens, x.shape[1], ctx.act_dtype)
        if getattr(ctx.ws, "input_cast", None) != (x.data_ptr(), ctx.n_tokens, id(ctx)):
            ops.cast_rows(x, h, ctx.n_tokens)
        return h

    def _add_normed(self, norm, y, x, ctx: StepContext) -> None:
        if ctx.act_dtype == torch.bfloat16 and hasattr(norm, "groups"):
            norm(y, x, accumulate=True, also=ctx.ws.get("block_input", ctx.n_tokens, x.shape[1], ctx.act_dtype))
            ctx.ws.input_cast = (x.data_ptr(), ctx.n_tokens, id(ctx))
        else:
            norm(y, x, accumulate=True)
            ctx.ws.input_cast = None

    def forward(self, x: torch.Tensor, ctx: StepContext, view, writes_cache: bool = True) -> None:
        ctx.ws.row_stats.forget()
        y = ctx.ws.get("block_sublayer_out", ctx.n_tokens, x.shape[1], torch.float32)
        if self.mixer is not None:
            self.mixer.forward(self._input(x, ctx), y, ctx, view, writes_cache, accumulate=False)
            self._add_normed(self.norm1, y, x, ctx)
        if self.feed_forward is not None:
            self.feed_forward.forward(self._input(x, ctx), y, ctx, accumulate=False)
            self._add_normed(self.norm2, y, x, ctx)


@register_part("block", "hyper_connection")
class HyperConnectionBlock:
    """A pre-norm layer over a residual carried in `streams` rows per token, x_1 … x_S [tokens, S·width] float32.
    Sublayer q (the mixer, then the feed-forward) has read coefficients a_q [S], write coefficients b_q [S] and a mix
    matrix M_q [S, S] (indexed [from, to]):

        u = Σ_s a_q[s] · x_s,    y = sublayer_q(norm_q(u)),    x_t ← Σ_s M_q[s, t] · x_s + b_q[t] · y   (all t at once).

    The read and the norm are one kernel (`norm1`, `norm2`: "stream_rmsnorm" parts holding a_q); the sublayer leaves
    y in float32 scratch (`accumulate=False`); a write and the read that follows it (the mixer's write and the
    feed-forward's read; a layer's last write and the next layer's first read, where the model says that a block of this
    kind runs next) are one kernel.  The feed-forward may be absent."""

    leaves_row_stats = False

    def __init__(self, norm1, mixer, norm2, feed_forward, *, streams: int, mix1, out1, mix2=None, out2=None):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward
        self.streams = int(streams)
        self.mix1, self.out1, self.mix2, self.out2 = mix1, out1, mix2, out2
        if tuple(mix1.shape) != (streams, streams) or out1.numel() != streams:
            raise ValueError("HyperConnectionBlock: the mix is [streams, streams] and the write coefficients [streams]")
        if feed_forward is not None and (mix2 is None or out2 is None or norm2 is None):
            raise ValueError("HyperConnectionBlock: a feed-forward needs its norm and its coefficients")

    def cache_need(self):
        return self.mixer.cache_need()

    def _fusable_read(self, norm) -> bool:
        return getattr(norm, "coefficients", None) is not None and getattr(norm, "streams", 0) == self.streams

    def _write(self, x, mix, out, y, h, ctx: StepContext, reader) -> bool:
        """A sublayer's write; with `reader` (the norm part of whatever reads the streams next) the read in the same pass.
        Returns whether h holds that read."""
        from ..csrc import ops
        T = ctx.n_tokens
        if reader is not None and self._fusable_read(reader):
            ops.streams_write_read(x, self.streams, mix, out, y, reader.coefficients, reader.weight, reader.eps, h, T)
            return True
        ops.streams_write(x, self.streams, mix, out, y, T)
        return False

    def forward(self, x: torch.Tensor, ctx: StepContext, view, writes_cache: bool = True) -> None:
        T, d = ctx.n_tokens, x.shape[1] // self.streams
        ws = ctx.ws
        ws.row_stats.forget()
        h = ws.get("block_normed", T, d, ctx.act_dtype)
        y = ws.get("block_sublayer_out", T, d, torch.float32)
        # the block ahead may have left this block's first read with its last write
        if ws.normed_ready != (x.data_ptr(), T, id(ctx), id(self.norm1)):
            self.norm1(x, h, n_rows=T)
        ws.normed_ready = None
        # who reads the streams after this block's last write: the next block's first norm, if it is one of this kind
        nb = getattr(ctx, "next_block", None)
        after = nb.norm1 if isinstance(nb, HyperConnectionBlock) and nb.streams == self.streams else None
        self.mixer.forward(h, y, ctx, view, writes_cache, accumulate=False)
        if self.feed_forward is None:
            if self._write(x, self.mix1, self.out1, y, h, ctx, after):
                ws.normed_ready = (x.data_ptr(), T, id(ctx), id(after))
            return
        if not self._write(x, self.mix1, self.out1, y, h, ctx, self.norm2):
            self.norm2(x, h, n_rows=T)
        self.feed_forward.forward(h, y, ctx, accumulate=False)
        if self._write(x, self.mix2, self.out2, y, h, ctx, after):
            ws.normed_ready = (x.data_ptr(), T, id(ctx), id(after))
