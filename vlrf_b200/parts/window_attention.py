"""Softmax attention with grouped key/value heads, key and value sizes of their own, projection biases, a rotation of
part of every query and key head, and an optional sliding window.

    q = W_q h + b_q, k = W_k h + b_k, v = W_v h + b_v            (one product; float32 results)
    the first rot.dims entries of every query and key head rotated by position (a "qk" position part, or none)
    score(i, j) = (q_i · k_j) · scale,  j ≤ i, and i − j < window where there is a window
    out = W_o · concat_h softmax_j(score) v_j

Queries and keys have `dim` entries a head, values `vdim`; query head h reads key/value head h // (heads / kv_heads).
Rotation angles, scores and softmax are float32; keys and values lie in the paged cache in the activation dtype.

What else is a parameter, each absent by default:
  w_v None                 the values are the keys as projected, before norm and rotation (vdim = dim)
  w_k None (and w_v None)  the layer has no keys and values of its own: it attends another layer's cache with its own
                           queries (the model's schedule says whose), and keeps nothing
  qk_norm "head" | "all"   an RMS norm of queries and of keys ahead of the rotation: every head by itself with one weight
                           vector of `dim` entries for all heads, or the whole projection as one row; weights `q_norm`,
                           `k_norm`, `norm_eps`
  rotary                   its pairing (halves or neighbours), its frequency table and its factor on cosines and sines
  softcap c                score ← c · tanh(score / c) after the scale
  keep_first n             with a window: keys at positions below n stay visible to every later query
  sink [heads]             one more term exp(sink_h) in the denominator of head h's softmax, with nothing in the numerator
  w_gate [heads, width]    head h's result is multiplied by sigmoid(w_gate_h · input) ahead of the output projection; the
                           gate's logits ride in the input product as `heads` more float32 columns

The mixer is written in three stages so that another mixer can run it beside a second branch on the same input:
`in_weight` / `in_bias` (the rows of the input product), `core(proj, merged, …, factor)` (from the product's float32
result to the merged heads, times a factor, in the activation dtype; both may be column ranges of wider rows), and
`out_weight`.  `forward` chains the three."""
from __future__ import annotations

import torch

from ..cache import KVNeed
from ..csrc import ops
from .context import StepContext
from .registry import register_part


@register_part("mixer", "window_attention")
class WindowAttention:
    def __init__(self, w_q, w_k, w_v, w_out, *, n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float,
                 b_q=None, b_k=None, b_v=None, window: int = 0, rotary=None, qk_norm: str | None = None, q_norm=None, k_norm=None,
                 norm_eps: float = 0.0, softcap: float | None = None, keep_first: int = 0, sink=None, w_gate=None):
        H, G = int(n_heads), int(n_kv_heads)
        if H <= 0 or G <= 0 or H % G != 0:
            raise ValueError(f"window attention: {H} heads cannot share {G} key/value heads")
        self.own_kv, self.values_are_keys = w_k is not None, w_k is not None and w_v is None
        if w_k is None and w_v is not None:
            raise ValueError("window attention: values of its own need keys of its own")
        if self.values_are_keys and vdim != dim:
            raise ValueError(f"window attention: values that are the keys have their size ({dim}), not {vdim}")
        if tuple(w_q.shape)[0] != H * dim or (w_k is not None and tuple(w_k.shape)[0] != G * dim) \
                or (w_v is not None and tuple(w_v.shape)[0] != G * vdim):
            raise ValueError("window attention: W_q is [heads·dim, width], W_k [kv_heads·dim, width], W_v [kv_heads·vdim, width]")
        if w_out.shape[1] != H * vdim:
            raise ValueError("window attention: the output projection does not take the merged heads")
        if max(dim, vdim) > ops.WINDOW_HEAD_MAX:
            raise ValueError(f"window attention: head sizes {dim} and {vdim} are above the {ops.WINDOW_HEAD_MAX} the kernels take")
        if rotary is not None and (getattr(rotary, "where", None) != "qk" or rotary.dims > dim):
            raise ValueError("window attention: the rotation acts on queries and keys and on at most a head's entries")
        if window < 0:
            raise ValueError("window attention: a window is positive, or 0 for none")
        if keep_first < 0 or (keep_first > 0 and window <= 0):
            raise ValueError("window attention: keep_first goes with a window and is not negative")
        if softcap is not None and not softcap > 0.0:
            raise ValueError(f"window attention: a cap of {softcap} on the scores is not positive")
        if qk_norm not in (None, "head", "all"):
            raise ValueError(f"window attention: a norm of queries and keys is 'head' or 'all', not '{qk_norm}'")
        if qk_norm is not None:
            nq, nk = (dim, dim) if qk_norm == "head" else (H * dim, G * dim)
            if q_norm is None or q_norm.numel() != nq or (self.own_kv and (k_norm is None or k_norm.numel() != nk)) or not norm_eps > 0.0:
                raise ValueError("window attention: the norm of queries and keys needs its weights and a positive eps")
        if sink is not None and sink.numel() != H:
            raise ValueError("window attention: one sink per query head")
        if w_gate is not None and tuple(w_gate.shape) != (H, w_q.shape[1]):
            raise ValueError("window attention: the gate per head is [heads, width]")
        weights = [w_q] + ([w_k] if w_k is not None else []) + ([w_v] if w_v is not None else [])
        biases = [b_q] + ([b_k] if w_k is not None else []) + ([b_v] if w_v is not None else [])
        if any(b is not None for b in biases) and any(b is None for b in biases):
            raise ValueError("window attention: biases for all projections or for none")
        if w_gate is not None and b_q is not None:
            raise ValueError("window attention: a gate per head goes with projections without biases")
        self.n_heads, self.n_kv_heads, self.dim, self.vdim = H, G, int(dim), int(vdim)
        self.scale, self.window, self.rotary = float(scale), int(window), rotary
        self.qk_norm, self.norm_eps = qk_norm, float(norm_eps)
        self.q_norm = q_norm.float().contiguous() if qk_norm is not None else None
        self.k_norm = k_norm.float().contiguous() if qk_norm is not None and self.own_kv else None
        self.softcap, self.keep_first = float(softcap) if softcap is not None else 0.0, int(keep_first)
        self.sink = sink.float().contiguous() if sink is not None else None
        self.q_off, self.k_off = 0, H * dim
        self.v_off = self.k_off if self.values_are_keys else H * dim + G * dim
        width_kv = (G * dim if w_k is not None else 0) + (G * vdim if w_v is not None else 0)
        self.gate_off = H * dim + width_kv if w_gate is not None else None
        if w_gate is not None:
            weights.append(w_gate.to(w_q.dtype))
        self.in_weight = torch.cat(weights, dim=0).contiguous()
        self.in_bias = torch.cat([b.float() for b in biases]).contiguous() if b_q is not None else None
        self.in_width = self.in_weight.shape[0]
        self.out_weight = w_out
        self.merged_width = H * vdim

    def cache_need(self):
        """Keys and values per token; a layer without projections of its own states the need of the cache it reads (the
        model checks that the two agree) and writes nothing."""
        kind = "window" if self.window > 0 else "full"
        return KVNeed(self.n_kv_heads, self.dim, kind, self.window, v_dim=self.vdim if self.vdim != self.dim else 0,
                      keep_first=self.keep_first)

    fuses_norm = False
    leaves_row_stats = False

    def kernels(self, act_dtype: torch.dtype, block_tokens: int) -> dict:
        return ops.attention_window_kind(act_dtype, self.dim, self.vdim, self.n_heads, self.n_kv_heads)

    def core(self, proj, merged, ctx: StepContext, view, writes_cache: bool = True, factor: float = 1.0) -> None:
        T, H, G = ctx.n_tokens, self.n_heads, self.n_kv_heads
        if writes_cache and not self.own_kv:
            raise ValueError("window attention: a layer without keys and values of its own must read another layer's cache")
        q = ctx.ws.get("window_q", T, H * self.dim, ctx.act_dtype)
        freq = self.rotary.inv_freq if self.rotary is not None else None
        rot = self.rotary.dims if self.rotary is not None else 0
        ops.qkv_rope_append(proj, self.q_off, self.k_off, self.v_off, freq, rot, q, view.k, view.v, view.block_table, ctx.tok_slot,
                            ctx.tok_pos, T, H, G, self.dim, self.vdim, writes_cache and self.own_kv, ctx.dev_err, norm=self.qk_norm,
                            q_norm=self.q_norm, k_norm=self.k_norm, eps=self.norm_eps,
                            interleaved=bool(getattr(self.rotary, "interleaved", False)),
                            magnitude=float(getattr(self.rotary, "magnitude", 1.0)))
        ops.attention_window_step(q, view.k, view.v, view.block_table, merged, ctx, H, G, self.dim, self.vdim, self.scale,
                                  self.window, factor, softcap=self.softcap, keep_first=self.keep_first, sink=self.sink,
                                  # head h times sigmoid of its gate logit (a float32 column of the input product), applied by
                                  # the attention kernel where it writes the head's result
                                  gate=proj[:, self.gate_off:self.gate_off + H] if self.gate_off is not None else None)

    def forward(self, h, x: torch.Tensor, ctx: StepContext, view, writes_cache: bool = True, accumulate: bool = True) -> None:
        T = ctx.n_tokens
        proj = ctx.ws.get("window_in_proj", T, self.in_width, torch.float32)
        ops.linear(h, self.in_weight, self.in_bias, proj)
        merged = ctx.ws.get("attn_out", T, self.merged_width, ctx.act_dtype)
        self.core(proj, merged, ctx, view, writes_cache)
        ops.linear(merged, self.out_weight, None, x, residual=x if accumulate else None)
