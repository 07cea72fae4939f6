"""A feed-forward of routed experts.

Every token takes the `top` experts with the largest router logits z = h·W_routerᵀ + b (float32 sums; ties go to the
lower index), weighted by the softmax over the chosen logits alone.  An expert is a gated feed-forward without biases,
W_down (silu(W_gate h) · (W_up h)).  A shared expert of the same form, if there is one, runs for every token and is
added, multiplied by sigmoid(w_sg · h), one number per token.

What else is a parameter.  An expert without a gate (`w_gate=None`): W_down relu(W_up h)².  Routing by scores
(`scoring="softmax_all"`): s = softmax(z) over all router outputs; a token chooses by s + `correction` (a vector; the
weights do not see it) among the outputs of the `keep` best of `groups` equal groups of neighbours, a group's score
being its largest s + correction, and weighs the chosen by s · `weight_scale` without renormalizing.  Identity
experts (`n_identity`): the router's last n_identity outputs stand for experts without matrices that return their
input, so the router has n_identity more rows than there are expert matrices.  `scoring="sigmoid"`: the same rule with
s = sigmoid(z), each output by itself.  `gate="clamped"` (with `limit`, `gate_alpha`): an expert is
W_down (g · sigmoid(gate_alpha · g) · (u + 1)) with g = min(W_gate h, limit) and u = clamp(W_up h, −limit, limit).

Nothing is decided on the host: the router's kernel counts each expert's rows, the tokens' inputs are copied into a
buffer sorted by expert, and two grouped products (each row block with its expert's matrix) run over it with the gate
between them; a last kernel sums each token's experts with their weights.  So a step with this part launches the same
kernels whatever the tokens choose, and can be captured and replayed.  The shared gate's logit rides in the router's
product as one more row.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .context import StepContext
from .registry import register_part


@register_part("feed_forward", "routed_experts")
class RoutedExperts:
    def __init__(self, w_router, b_router, w_gate, w_up, w_down, *, top: int, shared=None, scoring: str = "softmax_chosen",
                 correction=None, groups: int = 1, keep: int = 1, weight_scale: float = 1.0, n_identity: int = 0,
                 gate: str = "silu", limit: float | None = None, gate_alpha: float = 1.0):
        """w_router [E + n_identity, width], b_router [E + n_identity] float32 or None; w_gate (or None), w_up [E, ff, width],
        w_down [E, width, ff]; shared: None or (w_gate [ffs, width], w_up [ffs, width], w_down [width, ffs], w_sg [1, width]
        or None); correction: float32 [E + n_identity] or None."""
        n_out, width = w_router.shape
        E = n_out - int(n_identity)
        if n_identity < 0 or E < 0 or (E == 0) != (w_up is None):
            raise ValueError("routed experts: the router has one row per expert matrix and one per identity expert")
        ff = w_up.shape[1] if w_up is not None else 0
        if E > 0:
            if w_up.shape[0] != E or w_up.shape[2] != width or (w_gate is not None and w_gate.shape != w_up.shape):
                raise ValueError("routed experts: the experts' gate and up matrices are [experts, ff, width]")
            if tuple(w_down.shape) != (E, width, ff):
                raise ValueError("routed experts: the experts' down matrices are [experts, width, ff]")
        if scoring not in ("softmax_chosen", "softmax_all", "sigmoid"):
            raise ValueError(f"routed experts: scoring '{scoring}' is none of 'softmax_chosen', 'softmax_all', 'sigmoid'")
        if gate not in ("silu", "clamped") or (gate == "clamped" and (w_gate is None or limit is None or not limit > 0.0)):
            raise ValueError("routed experts: the experts' gate is 'silu', or 'clamped' with gate matrices and a positive limit")
        self.gate, self.limit, self.gate_alpha = gate, float(limit) if limit is not None else 0.0, float(gate_alpha)
        if scoring == "softmax_chosen" and (n_identity or correction is not None or groups != 1 or weight_scale != 1.0):
            raise ValueError("routed experts: identity experts, a correction, groups and a weight scale belong to scoring 'softmax_all'")
        if groups < 1 or n_out % groups != 0 or not (1 <= keep <= groups):
            raise ValueError(f"routed experts: {n_out} router outputs cannot form {groups} equal groups of which {keep} are kept")
        if not (0 < top <= min(keep * (n_out // groups), 32)):
            raise ValueError(f"routed experts: a token takes 1…min(32, {keep * (n_out // groups)}) experts, not {top}")
        if n_out > ops.MOE_MAX_OUTPUTS:
            raise ValueError(f"routed experts: the router's kernel takes up to {ops.MOE_MAX_OUTPUTS} outputs, not {n_out}")
        if b_router is not None and scoring != "softmax_chosen":
            raise ValueError(f"routed experts: scoring '{scoring}' has a correction of the choice, not a bias of the logits")
        self.n_experts, self.n_outputs, self.n_identity, self.top, self.width, self.ff = E, n_out, int(n_identity), int(top), width, ff
        self.scoring, self.groups, self.keep, self.weight_scale = scoring, int(groups), int(keep), float(weight_scale)
        self.correction = None
        if scoring != "softmax_chosen":
            self.correction = (correction.float() if correction is not None
                               else torch.zeros(n_out, dtype=torch.float32, device=w_router.device)).contiguous()
            if tuple(self.correction.shape) != (n_out,):
                raise ValueError("routed experts: the correction has one number per router output")
        self.gated = w_gate is not None
        if E > 0:
            self.w_gate_up = (torch.cat([w_gate, w_up], dim=1) if self.gated else w_up).contiguous()   # [E, (2·)ff, width]
            self.w_down = w_down.contiguous()
        else:
            self.w_gate_up = self.w_down = None
        self.shared = None
        self.shared_gate = False
        w_r = w_router
        b_r = b_router if b_router is not None else torch.zeros(n_out, dtype=torch.float32, device=w_router.device)
        self._no_bias = b_router is None and shared is None
        if shared is not None:
            s_gate, s_up, s_down, s_sg = shared
            if s_gate.shape != s_up.shape or s_gate.shape[1] != width or tuple(s_down.shape) != (width, s_gate.shape[0]):
                raise ValueError("routed experts: the shared expert's matrices do not chain")
            self.shared = (torch.cat([s_gate, s_up], dim=0).contiguous(), s_down.contiguous(), s_gate.shape[0])
            if s_sg is not None:
                if tuple(s_sg.shape) != (1, width):
                    raise ValueError("routed experts: the shared expert's gate is one row of the model's width")
                w_r = torch.cat([w_router, s_sg.to(w_router.dtype)], dim=0)
                b_r = torch.cat([b_r, torch.zeros(1, dtype=torch.float32, device=b_r.device)])
                self.shared_gate = True
        # One product of the input gives the router's logits (with the shared gate's) and, for few rows (a decode
        # step), behind them the shared expert's gate and up rows, all float32; with many rows the shared expert's
        # are a product of their own in the activation dtype, half the bytes.
        self.n_logits = w_r.shape[0]
        if self.shared is not None:
            w_gu = self.shared[0]
            self.w_in = torch.cat([w_r, w_gu], dim=0).contiguous()
            self.b_in = torch.cat([b_r, torch.zeros(w_gu.shape[0], dtype=torch.float32, device=b_r.device)]).contiguous()
        else:
            self.w_in, self.b_in = w_r.contiguous(), b_r.contiguous()

    fuses_norm = False
    leaves_row_stats = False

    def forward(self, h, x: torch.Tensor, ctx: StepContext, norm=None, accumulate: bool = True) -> None:
        T, ws, act = ctx.n_tokens, ctx.ws, ctx.act_dtype
        E, top, width, ff = self.n_experts, self.top, self.width, self.ff
        P = T * top
        shared_apart = self.shared is not None and T > ops.SKINNY_MAX_ROWS
        n_in = self.n_logits if shared_apart else self.w_in.shape[0]
        inp = ws.get("moe_in_proj", T, n_in, torch.float32)
        ops.linear(h, self.w_in[:n_in], None if self._no_bias else self.b_in[:n_in], inp)
        z = inp
        ids = ws.get("moe_ids", T, top, torch.int32)
        rank = ws.get("moe_rank", T, top, torch.int32)
        row_of = ws.get("moe_row_of", T, top, torch.int32)
        wts = ws.get("moe_weights", T, top, torch.float32)
        gate = ws.get("moe_shared_gate", T, 1, torch.float32) if self.shared_gate else None
        counts = ws.get_zeroed("moe_counts", max(E, 1), torch.int32)
        offsets = ws.get("moe_offsets", 1, max(E, 1) + 1, torch.int32)
        if self.scoring != "softmax_chosen":
            ops.moe_route_scored(z, self.n_outputs, top, self.groups, self.keep, self.n_identity, self.weight_scale, self.correction,
                                 ctx.tok_slot, ids, wts, rank, counts, T, scoring="sigmoid" if self.scoring == "sigmoid" else "softmax")
        else:
            ops.moe_route(z, E, top, self.shared_gate, ctx.tok_slot, ids, wts, rank, gate, counts, T)
        ops.moe_plan(counts, offsets, max(E, 1))
        rows = ws.get("moe_sorted", P, width, act)
        ops.moe_gather(h, ids, rank, offsets, rows, row_of, T, top)
        out = ws.get("moe_expert_out", P, width, torch.float32)
        if E > 0:
            a = ws.get("moe_inner", P, ff, act)
            if self.gated:
                u = ws.get("moe_gate_up", P, 2 * ff, act)
                ops.linear_grouped(rows, self.w_gate_up, u, offsets, P)
                if self.gate == "clamped":
                    ops.gate_mul_clamped(u[:, :ff], u[:, ff:], a, self.limit, self.gate_alpha, P, ff)
                else:
                    ops.gate_mul(u[:, :ff], u[:, ff:], a, "silu", P, ff)
            else:
                ops.linear_grouped(rows, self.w_gate_up, a, offsets, P, act="relu2")     # (the activation in the product's epilogue)
            ops.linear_grouped(a, self.w_down, out, offsets, P)
        shared_out = None
        if self.shared is not None:
            w_gu, w_d, ffs = self.shared
            sa = ws.get("moe_shared_inner", T, ffs, act)
            if shared_apart:
                su = ws.get("moe_shared_gate_up", T, 2 * ffs, act)
                ops.linear(h, w_gu, None, su)
                ops.gate_mul(su[:, :ffs], su[:, ffs:], sa, "silu", T, ffs)
            else:
                at = self.n_logits
                ops.gate_mul(inp[:, at:at + ffs], inp[:, at + ffs:at + 2 * ffs], sa, "silu", T, ffs)
            shared_out = ws.get("moe_shared_out", T, width, torch.float32)
            ops.linear(sa, w_d, None, shared_out)
        if self.n_identity:
            ops.moe_combine(out, row_of, wts, top, shared_out, gate, x, T, residual=x if accumulate else None, ids=ids, h=h)
        else:
            ops.moe_combine(out, row_of, wts, top, shared_out, gate, x, T, residual=x if accumulate else None)
