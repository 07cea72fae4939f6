"""Norms.  A norm reads rows of the float32 residual stream and writes rows in the activation dtype."""
from __future__ import annotations

import torch

from ..cache import StateNeed
from ..csrc import ops
from .registry import register_part


@register_part("norm", "layernorm")
class LayerNorm:
    """y = (x − mean)·(1/sqrt(var + eps))·weight + bias over the last axis, biased variance, statistics
    in float32 (reference: include/model/ops.hpp:443-476)."""

    #: what a product kernel may compute in its own prologue instead of calling this norm: a mixer or feed-forward
    #: that is handed the norm looks here (and at weight / bias / eps), never at the class
    fusable_as = "layernorm"

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor, eps: float):
        if weight.shape != bias.shape or weight.dim() != 1:
            raise ValueError("LayerNorm: weight and bias are vectors of one length")
        self.weight, self.bias, self.eps = weight, bias, float(eps)
        self.width = weight.shape[0]

    def __call__(self, x: torch.Tensor, out: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        """out[r] = LN(x[rows[r]]) when `rows` is given, else row by row."""
        ops.layernorm(x, self.weight, self.bias, self.eps, out, rows)
        return out


@register_part("norm", "group_rmsnorm")
class GroupRMSNorm:
    """The row is cut into `groups` equal consecutive parts; each part is divided by sqrt(mean(part²) + eps) of its
    own, and the whole row is multiplied by weight.  One group is the plain RMS norm.  Sums and the division are
    float32.  `accumulate=True` adds the result to the (float32) output rows instead of replacing them, which is
    what a block needs that norms a sublayer's output before the residual sum.

    `offset` is added to the stored weight (1.0 where a checkpoint holds the offset from one, y = x̂ · (1 + w)), and
    `post_scale`, a vector, multiplies the normed row element by element (a layer scale on a sublayer's normed output);
    both are folded into one float32 factor per column when the part is made."""

    def __init__(self, weight: torch.Tensor, eps: float, groups: int = 1, offset: float = 0.0, post_scale: torch.Tensor | None = None):
        if weight.dim() != 1 or groups < 1 or weight.shape[0] % groups != 0:
            raise ValueError(f"GroupRMSNorm: {tuple(weight.shape)} weights cannot be cut into {groups} equal parts")
        if post_scale is not None and post_scale.shape != weight.shape:
            raise ValueError("GroupRMSNorm: the scale behind the norm has one number per column")
        self.stored_weight, self.offset, self.post_scale = weight, float(offset), post_scale
        if offset != 0.0 or post_scale is not None:
            weight = weight.float() + float(offset)
            if post_scale is not None:
                weight = weight * post_scale.float()
            weight = weight.contiguous()
        self.weight, self.eps, self.groups = weight, float(eps), int(groups)
        self.width = weight.shape[0]

    def __call__(self, x: torch.Tensor, out: torch.Tensor, rows: torch.Tensor | None = None, accumulate: bool = False,
                 also: torch.Tensor | None = None) -> torch.Tensor:
        """also: a bfloat16 tensor that receives the finished rows as well (what the next sublayer reads of them)."""
        ops.group_rmsnorm(x, self.weight, self.eps, self.groups, out, rows, accumulate, also=also)
        return out


@register_part("norm", "stream_rmsnorm")
class StreamSumRMSNorm:
    """The RMS norm of a weighted sum of a residual's streams: a row of x is `streams` rows of `width` numbers, and
    y = u / sqrt(mean(u²) + eps) · weight with u = Σ_s coefficients[s] · x_s (coefficients None: the plain sum, which is
    what a model's last norm reads of such a residual).  One stream without coefficients is the plain RMS norm."""

    def __init__(self, weight: torch.Tensor, eps: float, streams: int = 1, coefficients: torch.Tensor | None = None):
        if weight.dim() != 1 or streams < 1 or (coefficients is not None and coefficients.numel() != streams):
            raise ValueError("StreamSumRMSNorm: a weight vector, and one coefficient per stream")
        self.weight, self.eps, self.streams, self.coefficients = weight, float(eps), int(streams), coefficients
        self.width = weight.shape[0]

    def __call__(self, x: torch.Tensor, out: torch.Tensor, rows: torch.Tensor | None = None, n_rows: int | None = None) -> torch.Tensor:
        ops.streams_read_norm(x, self.streams, self.coefficients, self.weight, self.eps, out, rows, n_rows)
        return out


@register_part("norm", "rmsnorm_shift")
class ShiftedRMSNorm:
    """The plain RMS norm followed by a token shift: with n_t = x_t / sqrt(mean(x_t²) + eps) · weight,

        y_t = n_t + (n_(t−1) − n_t) · mu      (element by element; n_(−1) = 0),

    n_(t−1) being the normed row of the sequence's token before, as it was before any shift.  A step that does not bring
    that token finds its normed row in the sequence's state, so this norm keeps something per sequence and says so
    (`cache_need`): a float32 row held twice, read and written by the parity of the positions, so that a step of one
    token may run twice.  The block that owns the norm hands it the step and its state.  The norm, the difference and
    the sum are float32; y is rounded once to the activation dtype."""

    def __init__(self, weight: torch.Tensor, mu: torch.Tensor, eps: float):
        if weight.dim() != 1 or mu.shape != weight.shape:
            raise ValueError("ShiftedRMSNorm: the weight and the shift's coefficients are vectors of one length")
        self.weight, self.mu, self.eps = weight, mu, float(eps)
        self.width = weight.shape[0]

    def cache_need(self):
        return StateNeed((2, self.width), torch.float32)

    def __call__(self, x: torch.Tensor, out: torch.Tensor, *, ctx, state: torch.Tensor) -> torch.Tensor:
        ops.rmsnorm_shift(x, self.weight, self.mu, self.eps, state, ctx, out)
        return out
