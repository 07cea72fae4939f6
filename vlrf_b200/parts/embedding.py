"""Token embedding and the head that turns the last hidden rows into logits."""
from __future__ import annotations

import torch

from ..csrc import ops
from .context import StepContext


class TokenEmbedding:
    """x[t] = weight[token[t]], fused with a position encoding that acts at the embedding
    (reference: include/model/ops.hpp:615-626, include/model/transformer.hpp:340)."""

    def __init__(self, weight: torch.Tensor, position=None, norm=None, scale: float = 1.0, streams: int = 1, bigram=None):
        """norm: a norm part applied to the embedded rows in place (float32), or None.  scale: a factor on every
        embedded row.  streams: how many copies of the row the residual starts with (a residual carried in several
        streams, see parts/block.py); the rows this part writes are `out_width` = streams · width wide.
        bigram: None, or (table [buckets + 1, width], mul_prev, mul_cur): the row (token before · mul_prev + token ·
        mul_cur) mod buckets of the table is added to the scaled embedding (not scaled itself), the table's last row
        for a sequence's first token.  The token before is then part of what a sequence keeps: the part says so with
        `cache_need`, and the model hands it the state when it calls it."""
        self.weight = weight
        self.bigram = None
        if bigram is not None:
            table, mul_prev, mul_cur = bigram
            if table.dim() != 2 or table.shape[0] < 2 or table.shape[1] != weight.shape[1] or table.dtype != weight.dtype:
                raise ValueError("TokenEmbedding: the bigram table is [buckets + 1, width] in the embedding's dtype")
            if norm is not None or streams != 1 or getattr(position, "where", None) == "embedding":
                raise ValueError("TokenEmbedding: a bigram table goes with one stream, no norm and no position table")
            buckets = int(table.shape[0]) - 1
            # (a multiplier enters the hash only through its remainder, which keeps every product inside 64 bits)
            self.bigram = (table, buckets, int(mul_prev) % buckets, int(mul_cur) % buckets)
        self.norm = norm
        self.vocab_size, self.width = weight.shape
        self.scale, self.streams = float(scale), int(streams)
        if self.streams < 1:
            raise ValueError("TokenEmbedding: at least one stream")
        if (self.scale != 1.0 or self.streams != 1) and (norm is not None or getattr(position, "where", None) == "embedding"):
            raise ValueError("TokenEmbedding: a scaled or copied embedding takes no norm and no position table")
        self.out_width = self.width * self.streams
        if position is not None and getattr(position, "where", None) == "embedding":
            if position.table.shape[1] != self.width or position.table.dtype != weight.dtype:
                raise ValueError("TokenEmbedding: the position table does not match the embedding")
            self.position = position
        else:
            self.position = None

    def cache_need(self):
        """What the embedding keeps per sequence: with a bigram table, the sequence's last token (held twice, by the
        parity of the sequence's length, so that a step of one token may run twice); else nothing."""
        if self.bigram is None:
            return None
        from ..cache import StateNeed
        return StateNeed((2,), torch.int32)

    @property
    def leaves_row_stats(self) -> bool:
        """The rows are written by a kernel that is handed the step's row statistics (see parts/block.py); a norm
        behind it rewrites them."""
        return self.norm is None and self.scale == 1.0 and self.streams == 1 and self.bigram is None

    def emit_decode(self, program, x: torch.Tensor) -> None:
        if self.scale != 1.0 or self.streams != 1 or self.bigram is not None:
            from .program import NotFusable
            raise NotFusable("a scaled or copied embedding, or one with a bigram table, is not an operation of the decode program")
        if self.norm is not None:
            from .program import NotFusable
            raise NotFusable("an embedding with a norm behind it is not an operation of the decode program")
        program.embed(self.weight, self.position.table if self.position is not None else None, x)

    def __call__(self, ctx: StepContext, x: torch.Tensor, state: torch.Tensor | None = None) -> torch.Tensor:
        if self.bigram is not None:
            if state is None:
                raise ValueError("TokenEmbedding: a bigram table needs the sequences' kept tokens")
            table, buckets, mul_prev, mul_cur = self.bigram
            ctx.ws.row_stats.forget()
            # In the bfloat16 engine the kernel also leaves the rows' rounding where a block that reads the residual itself
            # looks for it (`Workspace.input_cast`), which spares the first layer a cast kernel.
            also = ctx.ws.get("block_input", ctx.n_tokens, x.shape[1], ctx.act_dtype) if ctx.act_dtype == torch.bfloat16 else None
            ops.embed_bigram(self.weight, table, buckets, mul_prev, mul_cur, self.scale, state, ctx, x, also=also)
            if also is not None:
                ctx.ws.input_cast = (x.data_ptr(), ctx.n_tokens, id(ctx))
            return x
        if self.scale != 1.0 or self.streams != 1:
            ctx.ws.row_stats.forget()
            ops.embed_streams(self.weight, ctx.tokens, x, self.streams, self.scale, ctx.dev_err)
            return x
        table = self.position.table if self.position is not None else None
        ops.embed(self.weight, table, ctx.tokens, ctx.tok_pos if table is not None else None, x, ctx.dev_err,
                  stats=ctx.ws.row_stats)
        if self.norm is not None:
            ctx.ws.row_stats.forget()
            self.norm(x, x)
        return x


class LMHead:
    """logits = h · weightᵀ, float32, no bias; a tied head is given the embedding's weight
    (reference: include/model/transformer.hpp:413-414, :298-300).  With `softcap` = c the logits are then squashed,
    c · tanh(logits / c); with `scale` they are multiplied by it first."""

    def __init__(self, weight: torch.Tensor, softcap: float | None = None, scale: float = 1.0):
        self.weight = weight
        self.scale = float(scale)
        self.vocab_size, self.width = weight.shape
        if softcap is not None and not softcap > 0.0:
            raise ValueError(f"LMHead: a soft cap of {softcap} is not positive")
        self.softcap = float(softcap) if softcap is not None else None

    def emit_decode(self, program, x: torch.Tensor, norm, logits: torch.Tensor) -> None:
        """logits = norm(x) · weightᵀ for every row of the program."""
        from .program import NotFusable, norm_terms
        if self.softcap is not None or self.scale != 1.0:
            raise NotFusable("a head with a soft cap or a scale is not an operation of the decode program")
        program.product(x, self.weight, None, logits, norm=norm_terms(norm))

    def __call__(self, h: torch.Tensor, logits: torch.Tensor, n_rows: int) -> torch.Tensor:
        ops.linear(h, self.weight, None, logits, rows=n_rows)
        if self.scale != 1.0:
            ops.scale_values(logits, n_rows, self.scale)
        if self.softcap is not None:
            ops.softcap(logits, n_rows, self.softcap)
        return logits
