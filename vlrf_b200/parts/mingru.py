"""A gated recurrence whose gates read only the current token (the "minGRU" form).

One product of the layer's input gives, per token, three rows of `width` numbers: the gate's logits a (with a bias), the
candidate's input u (with a bias) and the output gate's logits g.  Element by element along a sequence

    z = sigmoid(a),   c = u + 1/2 where u ≥ 0 and sigmoid(u) below,   S_t = (1 − z) · S_(t−1) + z · c,   S_(−1) = 0,

and the mixer's output is W_o (S_t · g · sigmoid(g)).  Gates, candidates, the recurrence and its state are float32 in
every engine; the product's operands are in the activation dtype with float32 results.

Per sequence the mixer keeps S: one float32 row, held twice (`StateNeed((2, width))`; the kernel reads the copy of the
parity of the position a step begins at and writes that of the position it ends at, so a step of one token may run twice).
"""
from __future__ import annotations

import torch

from ..cache import StateNeed
from ..csrc import ops
from .context import StepContext
from .registry import register_part


@register_part("mixer", "mingru")
class MinGRUMixer:
    def __init__(self, w_z, b_z, w_x, b_x, w_g, w_out):
        """w_z, w_x, w_g [width, model width]; b_z, b_x float32 [width] or None; w_out [model width, width]."""
        W = w_z.shape[0]
        if w_x.shape != w_z.shape or w_g.shape != w_z.shape or w_out.shape[1] != W:
            raise ValueError("minGRU mixer: the three input matrices are [width, model width] and the output matrix takes the state")
        for b in (b_z, b_x):
            if b is not None and tuple(b.shape) != (W,):
                raise ValueError("minGRU mixer: a bias has one number per channel of the state")
        self.width = int(W)
        self.in_weight = torch.cat([w_z, w_x, w_g], dim=0).contiguous()
        zeros = torch.zeros(W, dtype=torch.float32, device=w_z.device)
        self.in_bias = torch.cat([(b_z if b_z is not None else zeros).float(), (b_x if b_x is not None else zeros).float(),
                                  zeros]).contiguous()
        self.out_weight = w_out

    def cache_need(self):
        return StateNeed((2, self.width), torch.float32)

    fuses_norm = False
    leaves_row_stats = False

    def forward(self, h, x: torch.Tensor, ctx: StepContext, view, writes_cache: bool = True, accumulate: bool = True) -> None:
        if not writes_cache:
            raise ValueError("minGRU mixer: a layer cannot read another layer's state")
        T, W = ctx.n_tokens, self.width
        proj = ctx.ws.get("mingru_in_proj", T, 3 * W, torch.float32)
        ops.linear(h, self.in_weight, self.in_bias, proj)
        gated = ctx.ws.get("mingru_gated", T, W, ctx.act_dtype)
        ops.mingru_scan(proj, 0, W, 2 * W, W, view.state, ctx, gated)
        ops.linear(gated, self.out_weight, None, x, residual=x if accumulate else None)
