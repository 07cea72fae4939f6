"""Attention whose cache holds one latent per token instead of keys and values.

A token's cache row is [c | r]: the normed latent c (`kv_rank` numbers), from which every head's unrotated key and
its value are linear maps (k_h = Uk_h c, v_h = Uv_h c), and optionally a rotated key part r (`rot_dim` numbers) that
all heads share.  Per head

    score(p, j) = (q_h(p) · Uk_h c_j + qr_h(p) · r_j) · scale,     out_h(p) = Uv_h Σ_j softmax_j(score) c_j.

The kernels never form keys or values: the query is carried into the latent space (q'_h = Uk_hᵀ q_h, a product per
head), every head attends the rows themselves, and the head's result is carried back by Uv_h (another product per
head).  That is the same arithmetic with the sums taken in another order.

What is a parameter: how queries are made (directly, h·W_qᵀ, or through a latent of their own, RMSnorm(h·W_dqᵀ)·W_uqᵀ);
the rotated part and its rotation (a position part that acts on q/k, with the pairing it names, or none); a sigmoid
gate on the merged heads (W_g, from the same input: a row per merged column, or a row per head); whether the layer owns a cache row (W_dkv and its norm) or reads another layer's, as the
model's schedule says (`writes_cache=False`: it then has no W_dkv and uses the rows as they lie in the cache).
Norms, rotation angles, scores and softmax are float32; products take operands in the activation dtype.
"""
from __future__ import annotations

import torch

from ..cache import LatentNeed
from ..csrc import ops
from .context import StepContext
from .registry import register_part


@register_part("mixer", "latent_attention")
class LatentAttention:
    def __init__(self, *, n_heads: int, dim: int, vdim: int, kv_rank: int, rot_dim: int = 0, scale: float,
                 w_uk, w_uv, w_out, w_q=None, w_dq=None, dq_norm=None, w_uq=None, w_dkv=None, dkv_norm=None,
                 w_gate=None, rotary=None, eps: float = 1e-5, window: int = 0):
        H, C, R = int(n_heads), int(kv_rank), int(rot_dim)
        per_q = dim + R
        if (w_q is None) == (w_dq is None):
            raise ValueError("latent attention: queries come from W_q or from W_dq, its norm and W_uq, not both or neither")
        if w_q is not None and tuple(w_q.shape)[0] != H * per_q:
            raise ValueError(f"latent attention: W_q has {w_q.shape[0]} rows, {H * per_q} expected")
        if w_dq is not None:
            if dq_norm is None or w_uq is None or w_uq.shape[1] != w_dq.shape[0] or dq_norm.shape[0] != w_dq.shape[0]:
                raise ValueError("latent attention: the query latent, its norm and W_uq do not chain")
            if w_uq.shape[0] != H * per_q:
                raise ValueError(f"latent attention: W_uq has {w_uq.shape[0]} rows, {H * per_q} expected")
        if tuple(w_uk.shape) != (H * dim, C) or tuple(w_uv.shape) != (H * vdim, C):
            raise ValueError("latent attention: W_uk is [heads·dim, kv_rank] and W_uv [heads·vdim, kv_rank]")
        if w_out.shape[1] != H * vdim:
            raise ValueError("latent attention: the output projection does not take the merged heads")
        if w_dkv is not None and (w_dkv.shape[0] != C + R or dkv_norm is None or dkv_norm.shape[0] != C):
            raise ValueError(f"latent attention: W_dkv has kv_rank + rot_dim = {C + R} rows and a norm weight of {C}")
        if w_gate is not None and w_gate.shape[0] not in (H * vdim, H):
            raise ValueError("latent attention: the gate has one row per merged column, or one per head")
        if R > 0:
            if rotary is None or getattr(rotary, "where", None) != "qk" or rotary.dims > R:
                raise ValueError("latent attention: a rotated part needs a rotation of at most its own size")
        if C > ops.LATENT_MAX_RANK:
            raise ValueError(f"latent attention: a latent of {C} numbers is wider than the {ops.LATENT_MAX_RANK} the kernels hold")
        self.n_heads, self.dim, self.vdim, self.kv_rank, self.rot_dim = H, int(dim), int(vdim), C, R
        self.scale, self.eps, self.window = float(scale), float(eps), int(window)
        self.w_q, self.w_dq, self.dq_norm, self.w_uq = w_q, w_dq, dq_norm, w_uq
        self.w_dkv, self.dkv_norm, self.w_gate, self.w_out = w_dkv, dkv_norm, w_gate, w_out
        self.rotary = rotary if R > 0 else None
        # merged columns that share one gate logit: 1 (a gate per column) or vdim (a gate per head)
        self.gate_per = 1 if w_gate is None or w_gate.shape[0] == H * vdim else int(vdim)
        # Uk per head, transposed once: [H, kv_rank, dim], the operand that carries a head's query into latent space;
        # Uv per head as it is stored: [H, vdim, kv_rank]
        self.w_uk_t = w_uk.view(H, dim, C).transpose(1, 2).contiguous()
        self.w_uv = w_uv.view(H, vdim, C)
        # as stored, [H·dim, kv_rank] above [H·vdim, kv_rank]: one product forms a step's keys and values
        self.w_ukv_rows = torch.cat([w_uk, w_uv], dim=0).contiguous()
        # Everything that is a product of the layer's input with float32 results wanted is one product: the queries
        # (or their latent), the cache row before its norm and rotation, the gate's logits.  (Queries that are used as
        # they come, without a rotated part or a latent, stay a product of their own in the activation dtype.)
        first = w_dq if w_dq is not None else (w_q if R > 0 else None)
        parts, self._cols, at = [], {}, 0
        for name, m in (("q", first), ("kv", w_dkv), ("gate", w_gate)):
            if m is not None:
                parts.append(m)
                self._cols[name] = (at, at + m.shape[0])
                at += m.shape[0]
        self.w_in = torch.cat(parts, dim=0).contiguous() if parts else None

    def cache_need(self):
        if self.window > 0:
            return LatentNeed(self.kv_rank + self.rot_dim, "window", self.window)
        return LatentNeed(self.kv_rank + self.rot_dim)

    fuses_norm = False
    leaves_row_stats = False

    def kernels(self, act_dtype: torch.dtype, block_tokens: int) -> dict:
        kind = ops.attention_latent_kind(act_dtype, self.kv_rank, self.rot_dim)
        return {"prompt": kind["prompt"], "decode": kind["decode"]}

    def forward(self, h, x: torch.Tensor, ctx: StepContext, view, writes_cache: bool = True, accumulate: bool = True) -> None:
        T, ws, act = ctx.n_tokens, ctx.ws, ctx.act_dtype
        H, dim, vdim, C, R = self.n_heads, self.dim, self.vdim, self.kv_rank, self.rot_dim
        D = C + R
        inv_freq = self.rotary.inv_freq if self.rotary is not None else None
        rot_dims = self.rotary.dims if self.rotary is not None else 0
        pairs = bool(getattr(self.rotary, "interleaved", False))
        if writes_cache and self.w_dkv is None:
            raise ValueError("latent attention: a layer without W_dkv reads another layer's cache and cannot write one")
        # few rows (a decode step): the gate's logits ride in the same product, as float32; many rows: they are a
        # product of their own in the activation dtype, half the bytes
        # (a gate per head is a handful of columns and always rides along)
        proj, gate_apart = None, self.w_gate is not None and T > ops.SKINNY_MAX_ROWS and self.gate_per == 1
        if self.w_in is not None:
            n_in = self._cols["gate"][0] if gate_apart else self.w_in.shape[0]
            if n_in > 0:
                proj = ws.get("latent_in_proj", T, n_in, torch.float32)
                ops.linear(h, self.w_in[:n_in], None, proj)

        def cols(name):
            a, b = self._cols[name]
            return proj[:, a:b]

        if writes_cache:
            ops.latent_append(cols("kv"), C, R, self.dkv_norm, self.eps, inv_freq, rot_dims, view.rows, view.block_table,
                              ctx.tok_slot, ctx.tok_pos, T, ctx.dev_err, interleaved=pairs)
        # A prompt step whose sequences all begin at position 0 holds every key and value it needs itself: they are
        # formed (two products of the step's latents) and attended as plain rows, which takes (dim + R) + vdim
        # multiplications per query, key and head instead of the latent-space form's (C + R) + C.  Every other step
        # (a prompt's later portions, decode steps, mixed steps) attends the cache rows in latent space.
        as_rows = (ctx.max_new > 1 and self.window == 0 and len(ctx.host_seq_pos0) == ctx.n_seqs
                   and not any(ctx.host_seq_pos0) and ops.attention_rows_takes(act, dim, R, vdim, H))
        # queries: per head [dim | R]
        qp = ws.get("latent_qr", T, H * R, act) if as_rows and R > 0 else (None if as_rows else ws.get("latent_qp", T, H * D, act))
        q_c = 0 if as_rows else C                             # columns ahead of the rotated part in a head's row of qp
        qn = ws.get("latent_qn", T, H * dim, act)
        if self.w_dq is not None:
            cq = ws.get("latent_cq", T, self.w_dq.shape[0], act)
            ops.group_rmsnorm(cols("q"), self.dq_norm, self.eps, 1, cq)
            if R == 0:
                ops.linear(cq, self.w_uq, None, qn)
            else:
                q32 = ws.get("latent_q32", T, H * (dim + R), torch.float32)
                ops.linear(cq, self.w_uq, None, q32)
                ops.latent_q_rows(q32, H, dim, R, inv_freq, rot_dims, ctx.tok_pos, qn, qp, q_c, T, interleaved=pairs)
        elif R == 0:
            ops.linear(h, self.w_q, None, qn)
        else:
            ops.latent_q_rows(cols("q"), H, dim, R, inv_freq, rot_dims, ctx.tok_pos, qn, qp, q_c, T, interleaved=pairs)
        merged = ws.get("attn_out", T, H * vdim, act)
        if as_rows:
            rows_c = ws.get("latent_step_c", T, C, act)
            rows_r = ws.get("latent_step_r", T, R, act) if R > 0 else None
            ops.latent_gather(view.rows, C, R, view.block_table, ctx.tok_slot, ctx.tok_pos, rows_c, rows_r, T, ctx.dev_err)
            kv = ws.get("latent_keys_values", T, H * (dim + vdim), act)
            ops.linear(rows_c, self.w_ukv_rows, None, kv)
            ops.attention_rows(qn, qp, kv[:, :H * dim], rows_r, kv[:, H * dim:], ctx.seq_start, merged, ctx.n_seqs, ctx.max_new, H, dim, R, vdim, self.scale)
        else:
            ops.linear_heads(qn.view(T, H, dim), self.w_uk_t, qp.view(T, H, D)[:, :, :C], T)
            o = ws.get("latent_o", T, H * C, act)
            ops.attention_latent(qp, view.rows, C, R, view.block_table, ctx.tok_slot, ctx.tok_pos, o, T, H, self.scale,
                                 self.window, ctx.dev_err, ctx=ctx)
            ops.linear_heads(o.view(T, H, C), self.w_uv, merged.view(T, H, vdim), T)
        if gate_apart:
            g = ws.get("latent_gate", T, H * vdim, act)
            ops.linear(h, self.w_gate, None, g)
            ops.gate_mul(g, merged, merged, "sigmoid", T, H * vdim)
        elif self.w_gate is not None:
            ops.gate_mul(cols("gate"), merged, merged, "sigmoid", T, H * vdim, per=self.gate_per)
        ops.linear(merged, self.w_out, None, x, residual=x if accumulate else None)
